// C ABI of the library (see include/hf2q_cuda.h): argument validation, routing between the
// kernels, status handling.  Host code only; mirrors the checks hf2q performs before it calls
// mlx-native (shape and type allow-lists, src/inference/models/qwen35/weight_loader.rs:1059-1079;
// unsupported type is an error, src/serve/forward_mlx.rs:9647-9651).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <new>

#include "common.cuh"
#include "kernels.h"

using namespace hf2q;

struct hf2q_ctx {
    int device = -1;
    DeviceInfo dev{};
    uint32_t* status = nullptr;        // device status word
    uint64_t launches = 0;
    bool fp32_matvec = false;          // HF2Q_CUDA_F32_MATVEC=1: CUDA-core fp32 mat-vec only
    long long wait_limit = 1ll << 31;  // clock ticks a device-side wait for another GPU may take (about a second)
    // partial sums of the mat-vec's split-k form (rows too long for the activation panel); one buffer per
    // context, used by one launch at a time in stream order (a context serves one thread and stream at a time)
    float* splitk = nullptr;
    static constexpr uint64_t SPLITK_BYTES = 8ull << 20;
    uint32_t* misc = nullptr;          // 1 KiB of zero-initialised words: arrival counter and candidates of the arg-max
    // staging for the *_host convenience calls
    // A ring of device staging buffers and three streams: copy-in on in_stream, kernels on
    // host_stream, copy-out on out_stream, so that the copy-in of later calls, the kernel of call i
    // and the copy-out of earlier calls all overlap (the two copy directions use different copy
    // engines).  Slot i % HOST_SLOTS is reused by call i + HOST_SLOTS: its copy-in waits for the
    // slot's previous kernel (`computed`), its kernel for the slot's previous copy-out (`drained`).
    struct HostSlot {
        void* x = nullptr;  size_t x_bytes = 0;
        float* y = nullptr; size_t y_bytes = 0;
        cudaEvent_t loaded = nullptr, computed = nullptr, drained = nullptr;
        bool used = false;
    };
    static constexpr int HOST_SLOTS = 8;
    HostSlot hslot[HOST_SLOTS];
    uint32_t hnext = 0;
    cudaStream_t out_stream = nullptr, in_stream = nullptr;
    void* pin_x = nullptr;    size_t pin_x_bytes = 0;
    float* pin_y = nullptr;   size_t pin_y_bytes = 0;
    void* ws = nullptr;       size_t ws_bytes = 0;
    cudaStream_t host_stream = nullptr;
    // staging of hf2q_cuda_qmatmul_host_batch: one x and one y buffer for the whole batch, one event pair per group
    void* bx = nullptr;       size_t bx_bytes = 0;
    void* by = nullptr;       size_t by_bytes = 0;
    std::vector<cudaEvent_t> b_loaded, b_computed;
    cudaEvent_t b_all_computed = nullptr, b_all_drained = nullptr;
    bool b_used = false;
    // a batch that comes a second time unchanged (same items, same staging) is captured into a CUDA graph and replayed
    uint64_t b_last_key = 0, b_graph_key = 0, b_nograph_key = 0;
    cudaGraphExec_t b_graph = nullptr;
    uint64_t b_graph_launches = 0;
    cudaEvent_t b_fork = nullptr, b_join_in = nullptr, b_join_out = nullptr;
    char err[512] = {0};
};

namespace hf2q {
uint32_t* ctx_status_word(hf2q_ctx* ctx) { return ctx ? ctx->status : nullptr; }
// records `msg` as the context's last error and returns `code` (for the library's other translation units)
int32_t ctx_fail(hf2q_ctx* ctx, int32_t code, const char* msg) {
    if (ctx) snprintf(ctx->err, sizeof ctx->err, "%s", msg);
    return code;
}
}  // namespace hf2q

namespace {

int32_t fail(hf2q_ctx* ctx, int32_t code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof ctx->err, fmt, ap);
        va_end(ap);
    }
    return code;
}
int32_t cuda_fail(hf2q_ctx* ctx, cudaError_t e, const char* what) {
    const int32_t code = e == cudaErrorMemoryAllocation ? HF2Q_ERR_OUT_OF_MEMORY : HF2Q_ERR_CUDA;
    return fail(ctx, code, "%s: %s", what, cudaGetErrorString(e));
}

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    // (switching costs about a microsecond even to the current device, so it is done only when needed)
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev == dev) { ok = true; prev = -1; }
        else ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

size_t dtype_size(uint32_t dt) { return dt == HF2Q_DT_F32 ? 4 : 2; }

int32_t check_matmul_shape(hf2q_ctx* ctx, uint32_t type, uint32_t n, uint32_t k, const char* who) {
    if (!type_supported(type)) return fail(ctx, HF2Q_ERR_UNSUPPORTED_TYPE, "%s: type %u is not one of Q4_0/Q4_1/Q5_0/Q5_1/Q8_0/Q4_K/Q5_K/Q6_K/IQ4_NL/MLX_AFFINE4_GS32", who, type);
    const BlockGeom g = block_geom(type);
    if (n == 0 || k == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: n=%u k=%u must be non-zero", who, n, k);
    if (k % g.elems) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: k=%u is not a multiple of the %u-element block", who, k, g.elems);
    return HF2Q_OK;
}

int32_t grow(hf2q_ctx* ctx, void** p, size_t* have, size_t want, bool pinned) {
    if (*have >= want) return HF2Q_OK;
    if (*p) { pinned ? cudaFreeHost(*p) : cudaFree(*p); *p = nullptr; *have = 0; }
    cudaError_t e = pinned ? cudaMallocHost(p, want) : cudaMalloc(p, want);
    if (e != cudaSuccess) return cuda_fail(ctx, e, pinned ? "cudaMallocHost" : "cudaMalloc");
    *have = want;
    return HF2Q_OK;
}

// y[m,n] for m activation rows through the mat-vec kernels, split into as many launches as the
// chosen kernel needs.  ids == nullptr: dense.
int32_t run_matvec(hf2q_ctx* ctx, cudaStream_t st, GemvArgs a, uint32_t m_total, const char* who) {
    const size_t xs = dtype_size(a.x_dtype);
    const bool mma = !ctx->fp32_matvec && gemv_mma_supported(a);
    uint32_t step = 8;
    if (mma) {
        step = gemv_mma_max_rows(a.type, a.k, a.x_dtype, ctx->dev);
        if (step == 0) step = 8;
    }
    const bool use_mma = mma && gemv_mma_max_rows(a.type, a.k, a.x_dtype, ctx->dev) > 0;
    const uint8_t* x0 = static_cast<const uint8_t*>(a.x);
    float* y0 = a.y;
    const float* r0 = a.residual;
    for (uint32_t m0 = 0; m0 < m_total; m0 += step) {
        a.m = (m_total - m0) < step ? (m_total - m0) : step;
        a.x = x0 + static_cast<size_t>(m0) * a.k * xs;
        a.y = y0 + static_cast<size_t>(m0) * a.n;
        if (r0) a.residual = r0 + static_cast<size_t>(m0) * a.n;
        cudaError_t e;
        int nl = 1;
        a.splitk_scratch = ctx->splitk;
        a.splitk_bytes = hf2q_ctx::SPLITK_BYTES;
        a.n_launches = &nl;
        if (use_mma) e = launch_gemv_mma(a, ctx->dev, st);
        else e = launch_gemv(a, ctx->dev, st, &nl);
        if (e != cudaSuccess) return cuda_fail(ctx, e, who);
        ctx->launches += nl;
    }
    return HF2Q_OK;
}

}  // namespace

extern "C" {

HF2Q_API const char* hf2q_cuda_version(void) { return "hf2q-cuda 0.1 (sm_100a)"; }

HF2Q_API const char* hf2q_cuda_strerror(int32_t s) {
    switch (s) {
        case HF2Q_OK: return "ok";
        case HF2Q_ERR_INVALID_ARGUMENT: return "invalid argument";
        case HF2Q_ERR_UNSUPPORTED_TYPE: return "unsupported ggml type";
        case HF2Q_ERR_CUDA: return "CUDA runtime error";
        case HF2Q_ERR_WORKSPACE: return "workspace missing or too small";
        case HF2Q_ERR_TIMEOUT: return "device-side wait timed out";
        case HF2Q_ERR_OUT_OF_MEMORY: return "out of device memory";
        case HF2Q_ERR_NO_DEVICE: return "no usable CUDA device";
        default: return "unknown status";
    }
}

HF2Q_API const char* hf2q_cuda_last_error(const hf2q_ctx* ctx) { return ctx ? ctx->err : "null context"; }

HF2Q_API int32_t hf2q_cuda_ctx_create(int32_t device, hf2q_ctx** out) {
    if (!out) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) { (void)cudaGetLastError(); return HF2Q_ERR_NO_DEVICE; }
    if (device < 0 || device >= count) return HF2Q_ERR_INVALID_ARGUMENT;
    hf2q_ctx* c = new (std::nothrow) hf2q_ctx();
    if (!c) return HF2Q_ERR_OUT_OF_MEMORY;
    c->device = device;
    DeviceGuard g(device);
    cudaDeviceProp prop{};
    if (!g.ok || cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return HF2Q_ERR_CUDA; }
    if (prop.major < 10) { delete c; return HF2Q_ERR_NO_DEVICE; }   // kernels are sm_100a only
    c->dev.sm_count = prop.multiProcessorCount;
    c->dev.max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    if (cudaMalloc(&c->status, 256) != cudaSuccess || cudaMemset(c->status, 0, 256) != cudaSuccess ||
        cudaMalloc(&c->splitk, hf2q_ctx::SPLITK_BYTES) != cudaSuccess ||
        cudaMalloc(&c->misc, 1024) != cudaSuccess || cudaMemset(c->misc, 0, 1024) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->out_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->in_stream, cudaStreamNonBlocking) != cudaSuccess) {
        if (c->status) cudaFree(c->status);
        if (c->splitk) cudaFree(c->splitk);
        if (c->misc) cudaFree(c->misc);
        delete c;
        return HF2Q_ERR_CUDA;
    }
    // one knob, read once here and never on the launch path (the reference has the same kind of
    // switch for its mat-vec: HF2Q_F32_MATVEC, src/serve/forward_mlx.rs:9835)
    const char* env = getenv("HF2Q_CUDA_F32_MATVEC");
    c->fp32_matvec = env && env[0] == '1';
    *out = c;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_ctx_destroy(hf2q_ctx* ctx) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    DeviceGuard g(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->splitk) cudaFree(ctx->splitk);
    if (ctx->misc) cudaFree(ctx->misc);
    for (auto& hs : ctx->hslot) {
        if (hs.x) cudaFree(hs.x);
        if (hs.y) cudaFree(hs.y);
        if (hs.computed) cudaEventDestroy(hs.computed);
        if (hs.loaded) cudaEventDestroy(hs.loaded);
        if (hs.drained) cudaEventDestroy(hs.drained);
    }
    if (ctx->out_stream) cudaStreamDestroy(ctx->out_stream);
    if (ctx->in_stream) cudaStreamDestroy(ctx->in_stream);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->bx) cudaFree(ctx->bx);
    if (ctx->by) cudaFree(ctx->by);
    for (cudaEvent_t ev : ctx->b_loaded) cudaEventDestroy(ev);
    for (cudaEvent_t ev : ctx->b_computed) cudaEventDestroy(ev);
    if (ctx->b_all_computed) cudaEventDestroy(ctx->b_all_computed);
    if (ctx->b_all_drained) cudaEventDestroy(ctx->b_all_drained);
    if (ctx->b_graph) cudaGraphExecDestroy(ctx->b_graph);
    if (ctx->b_fork) cudaEventDestroy(ctx->b_fork);
    if (ctx->b_join_in) cudaEventDestroy(ctx->b_join_in);
    if (ctx->b_join_out) cudaEventDestroy(ctx->b_join_out);
    if (ctx->pin_x) cudaFreeHost(ctx->pin_x);
    if (ctx->pin_y) cudaFreeHost(ctx->pin_y);
    if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
    delete ctx;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_check_status(hf2q_ctx* ctx, void* stream) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    DeviceGuard g(ctx->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, ctx->status, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->status, 0, 4, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "status read-back");
    if (word & STATUS_WAIT_TIMEOUT) return fail(ctx, HF2Q_ERR_TIMEOUT, "a kernel gave up a bounded wait (status 0x%x)", word);
    if (word & STATUS_BAD_EXPERT_ID) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "ids[] held an expert index >= n_experts (status 0x%x)", word);
    if (word & STATUS_X_CLIPPED) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "an activation exceeded 65504 in magnitude and was clipped (status 0x%x)", word);
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_block_geometry(uint32_t t, uint32_t* be, uint32_t* bb) {
    if (!type_supported(t)) return HF2Q_ERR_UNSUPPORTED_TYPE;
    const BlockGeom g = block_geom(t);
    if (be) *be = g.elems;
    if (bb) *bb = g.bytes;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_row_bytes(uint32_t t, uint64_t k, uint64_t* out) {
    if (!out) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!type_supported(t)) return HF2Q_ERR_UNSUPPORTED_TYPE;
    const BlockGeom g = block_geom(t);
    if (k % g.elems) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = k / g.elems * g.bytes;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_expert_stride(uint32_t t, uint64_t rows, uint64_t cols, uint64_t* out) {
    uint64_t rb = 0;
    const int32_t rc = hf2q_cuda_row_bytes(t, cols, &rb);
    if (rc) return rc;
    *out = rows * rb;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_upload_blocks(hf2q_ctx* ctx, const void* host, uint64_t nbytes, void** dev_out) {
    if (!ctx || !host || !dev_out || nbytes == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "upload_blocks: null pointer or zero length");
    DeviceGuard g(ctx->device);
    void* d = nullptr;
    // 16 spare bytes keep 16-byte vector reads of the final partial chunk inside the allocation
    cudaError_t e = cudaMalloc(&d, nbytes + 16);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "upload_blocks: cudaMalloc");
    e = cudaMemcpy(d, host, nbytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(d); return cuda_fail(ctx, e, "upload_blocks: cudaMemcpy"); }
    *dev_out = d;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_free(hf2q_ctx* ctx, void* p) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    DeviceGuard g(ctx->device);
    const cudaError_t e = cudaFree(p);
    return e == cudaSuccess ? HF2Q_OK : cuda_fail(ctx, e, "cudaFree");
}

HF2Q_API int32_t hf2q_cuda_dequantize(hf2q_ctx* ctx, void* stream, const void* w, uint32_t type, uint64_t n,
                                      uint64_t k, void* out, uint32_t out_dtype) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!w || !out) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "dequantize: null pointer");
    if (!type_supported(type)) return fail(ctx, HF2Q_ERR_UNSUPPORTED_TYPE, "dequantize: ggml type %u unsupported", type);
    if (out_dtype > HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "dequantize: out_dtype %u", out_dtype);
    const BlockGeom g = block_geom(type);
    if (k == 0 || k % g.elems) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "dequantize: k=%llu not a multiple of %u", (unsigned long long)k, g.elems);
    if (reinterpret_cast<uintptr_t>(w) % 2) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "dequantize: weight pointer must be 2-byte aligned");
    if (n == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_dequant(type, w, out, out_dtype, n * k, ctx->dev.sm_count, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "dequantize launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_affine_pack(hf2q_ctx* ctx, void* stream, const uint32_t* codes, const float* scales, const float* biases,
                                       uint32_t n, uint32_t k, uint32_t bits, uint32_t group_size, void* out_blocks) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!codes || !scales || !biases || !out_blocks) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "affine_pack: null pointer");
    if (bits != 4 || group_size != 32)
        return fail(ctx, HF2Q_ERR_UNSUPPORTED_TYPE, "affine_pack: only bits=4, group_size=32 (got bits=%u gs=%u)", bits, group_size);
    if (k == 0 || k % 32) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "affine_pack: k=%u must be a non-zero multiple of 32", k);
    if (reinterpret_cast<uintptr_t>(codes) % 16 || reinterpret_cast<uintptr_t>(out_blocks) % 8 || reinterpret_cast<uintptr_t>(scales) % 4 ||
        reinterpret_cast<uintptr_t>(biases) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "affine_pack: codes must be 16-byte, the output 8-byte, scales and biases 4-byte aligned");
    if (n == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_affine_pack(codes, scales, biases, static_cast<uint64_t>(n) * (k / 32), out_blocks, ctx->dev.sm_count,
                                             static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "affine_pack launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, uint32_t type,
                                                   uint32_t x_dtype, uint64_t* out) {
    (void)n; (void)x_dtype;
    if (!out) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!type_supported(type)) return HF2Q_ERR_UNSUPPORTED_TYPE;
    // m <= 8 (mat-vec) needs none; the tensor-core GEMM keeps an f16 copy of the activations
    *out = m > 8 ? gemm_tc_workspace_bytes(m, k) : 0;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w,
                                   float* y, uint32_t m, uint32_t n, uint32_t k, uint32_t type,
                                   void* workspace, uint64_t workspace_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul: null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul: x_dtype %u (want F32 or BF16)", x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, "qmatmul");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    if (reinterpret_cast<uintptr_t>(w) % 2 || reinterpret_cast<uintptr_t>(x) % dtype_size(x_dtype) || reinterpret_cast<uintptr_t>(y) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul: misaligned buffer");
    DeviceGuard dg(ctx->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // m > 8: tensor-core GEMM (the reference's MM_ROUTING_THRESHOLD, forward_mlx.rs:9800) when the
    // layout allows tensor-map copies; otherwise the mat-vec kernels, 8 rows at a time
    if (m > 8 && !ctx->fp32_matvec && gemm_tc_supported(type, w, n, k)) {
        const uint64_t need = gemm_tc_workspace_bytes(m, k);
        if (!workspace || workspace_bytes < need)
            return fail(ctx, HF2Q_ERR_WORKSPACE, "qmatmul: m=%u needs a workspace of %llu bytes (got %llu)", m,
                        (unsigned long long)need, (unsigned long long)workspace_bytes);
        if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul: workspace must be 256-byte aligned");
        int nl = 0;
        const cudaError_t e = launch_gemm_tc(type, w, x, x_dtype, y, m, n, k, workspace, ctx->status, ctx->dev.sm_count, st, &nl);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul (tensor-core GEMM) launch");
        ctx->launches += nl;
        return HF2Q_OK;
    }
    GemvArgs a{};
    a.w = w; a.x = x; a.y = y;
    a.x_dtype = x_dtype; a.type = type;
    a.n = n; a.k = k;
    a.slots = 1; a.top_k = 1; a.n_experts = 0;
    a.status = ctx->status;
    return run_matvec(ctx, st, a, m, "qmatmul launch");
}

// The O projection of a prefill chunk reading the attention output where flash attention wrote it:
// x is [k / head_dim heads][m][head_dim] (bf16 in the reference, f32 accepted as well).
HF2Q_API int32_t hf2q_cuda_qmatmul_perm021(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w, float* y,
                                           uint32_t m, uint32_t n, uint32_t k, uint32_t head_dim, uint32_t type, void* workspace,
                                           uint64_t workspace_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    const char* who = "qmatmul_perm021";
    if (!x || !w || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: x_dtype %u (want F32 or BF16)", who, x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, who);
    if (rc) return rc;
    if (head_dim == 0 || head_dim % 8 || k % head_dim)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: head_dim=%u must be a multiple of 8 that divides k=%u", who, head_dim, k);
    if (m == 0) return HF2Q_OK;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(y) % 4) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: misaligned buffer", who);
    if (ctx->fp32_matvec || !gemm_tc_supported(type, w, n, k))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: needs the tensor-core GEMM (16-byte aligned weight rows, k %% 256 == 0)", who);
    const uint64_t need = gemm_tc_workspace_bytes(m, k);
    if (!workspace || workspace_bytes < need)
        return fail(ctx, HF2Q_ERR_WORKSPACE, "%s: m=%u needs a workspace of %llu bytes (got %llu)", who, m, (unsigned long long)need,
                    (unsigned long long)workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: workspace must be 256-byte aligned", who);
    DeviceGuard dg(ctx->device);
    int nl = 0;
    const cudaError_t e = launch_gemm_tc(type, w, x, x_dtype, y, m, n, k, workspace, ctx->status, ctx->dev.sm_count,
                                         static_cast<cudaStream_t>(stream), &nl, 0, false, nullptr, head_dim);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_perm021 launch");
    ctx->launches += nl;
    return HF2Q_OK;
}

// A matrix whose row ranges use different block formats (the fused QKV tensor of a Q4_K_M model:
// Q and K rows Q4_K, V rows Q6_K): one call, one conversion of the activations, one launch per range,
// every range writing its own columns of the one output.
static int32_t segments_impl(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const hf2q_row_segment* segs, uint32_t n_segs,
                             float* y, uint32_t m, uint32_t k, void* workspace, uint64_t workspace_bytes, const float* norm_w, float norm_eps) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !segs || !y || n_segs == 0 || n_segs > 16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: null pointer or n_segs=%u not in 1..16", n_segs);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: x_dtype %u (want F32 or BF16)", x_dtype);
    uint64_t n = 0;
    for (uint32_t i = 0; i < n_segs; ++i) {
        if (!segs[i].w) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: segment %u has no weights", i);
        const int32_t rc = check_matmul_shape(ctx, segs[i].ggml_type, segs[i].rows, k, "qmatmul_segments");
        if (rc) return rc;
        n += segs[i].rows;
    }
    if (n > 0xffffffffull) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: %llu rows", (unsigned long long)n);
    if (m == 0) return HF2Q_OK;
    if (reinterpret_cast<uintptr_t>(x) % dtype_size(x_dtype) || reinterpret_cast<uintptr_t>(y) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: misaligned buffer");
    DeviceGuard dg(ctx->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool gemm = m > 8 && !ctx->fp32_matvec;
    if (norm_w) {
        if (gemm || x_dtype != HF2Q_DT_F32 || m > 4)
            return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "norm_qmatmul_segments: the fused RMSNorm takes 1..4 f32 activation rows (m=%u, x_dtype=%u)", m, x_dtype);
        for (uint32_t i = 0; i < n_segs; ++i)
            if (!gemv_mma_norm_ok(segs[i].ggml_type, k, m, ctx->dev))
                return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "norm_qmatmul_segments: k=%u / type %u does not fit the fused RMSNorm (k <= 4096, k %% 256 == 0)", k, segs[i].ggml_type);
    }
    if (gemm) {
        const uint64_t need = gemm_tc_workspace_bytes(m, k);
        if (!workspace || workspace_bytes < need)
            return fail(ctx, HF2Q_ERR_WORKSPACE, "qmatmul_segments: m=%u needs a workspace of %llu bytes (got %llu)", m,
                        (unsigned long long)need, (unsigned long long)workspace_bytes);
        if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: workspace must be 256-byte aligned");
    }
    // every range must fit the kernel the row count selects: a detour for one range would need a second output layout
    uint32_t step = m;                  // activation rows per mat-vec launch (f32 rows take two MMA columns each)
    for (uint32_t i = 0; i < n_segs; ++i) {
        GemvArgs a{};
        a.w = segs[i].w; a.x = x; a.x_dtype = x_dtype; a.type = segs[i].ggml_type; a.n = segs[i].rows; a.k = k;
        bool ok;
        if (gemm) {
            ok = gemm_tc_supported(segs[i].ggml_type, segs[i].w, segs[i].rows, k);
        } else {
            const uint32_t rows = (!ctx->fp32_matvec && gemv_mma_supported(a)) ? gemv_mma_max_rows(segs[i].ggml_type, k, x_dtype, ctx->dev) : 0;
            ok = rows > 0;
            if (ok && rows < step) step = rows;
        }
        if (!ok) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_segments: segment %u (type %u, k=%u, m=%u) needs 16-byte aligned weight rows and k %% 256 == 0", i,
                             segs[i].ggml_type, k, m);
    }
    uint32_t col0 = 0;
    for (uint32_t i = 0; i < n_segs; ++i) {
        if (gemm) {
            int nl = 1;
            const cudaError_t e = launch_gemm_tc(segs[i].ggml_type, segs[i].w, x, x_dtype, y + col0, m, segs[i].rows, k, workspace, ctx->status,
                                                 ctx->dev.sm_count, st, &nl, static_cast<uint32_t>(n), i != 0);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_segments launch");
            ctx->launches += nl;
        } else {
            for (uint32_t m0 = 0; m0 < m; m0 += step) {
                GemvArgs a{};
                a.w = segs[i].w;
                a.x = static_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * k * dtype_size(x_dtype);
                a.y = y + static_cast<size_t>(m0) * n;
                a.x_dtype = x_dtype; a.type = segs[i].ggml_type;
                a.m = (m - m0) < step ? (m - m0) : step; a.n = segs[i].rows; a.k = k;
                a.slots = 1; a.top_k = 1; a.n_experts = 0;
                a.status = ctx->status;
                GatherArgs ga{};             // the one-rank form of the gathering store: columns [col0, col0 + rows) of a wider y
                ga.y_all[0] = a.y; ga.n_ranks = 1; ga.rank = 0; ga.n_total = static_cast<uint32_t>(n); ga.col0 = col0;
                ga.wait_limit = ctx->wait_limit;
                a.gather = &ga;
                a.norm_weight = norm_w;
                a.norm_eps = norm_eps;
                const cudaError_t e = launch_gemv_mma(a, ctx->dev, st);
                if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_segments launch");
                ctx->launches += 1;
            }
        }
        col0 += segs[i].rows;
    }
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_segments(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                            const hf2q_row_segment* segs, uint32_t n_segs, float* y, uint32_t m, uint32_t k,
                                            void* workspace, uint64_t workspace_bytes) {
    return segments_impl(ctx, stream, x, x_dtype, segs, n_segs, y, m, k, workspace, workspace_bytes, nullptr, 0.f);
}

HF2Q_API int32_t hf2q_cuda_norm_qmatmul_segments(hf2q_ctx* ctx, void* stream, const float* x, const float* norm_weight, float eps,
                                                 const hf2q_row_segment* segs, uint32_t n_segs, float* y, uint32_t m, uint32_t k) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!norm_weight) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "norm_qmatmul_segments: null norm weight");
    return segments_impl(ctx, stream, x, HF2Q_DT_F32, segs, n_segs, y, m, k, nullptr, 0, norm_weight, eps);
}

HF2Q_API int32_t hf2q_cuda_norm_supported(hf2q_ctx* ctx, uint32_t m, uint32_t k, uint32_t type) {
    if (!ctx || !type_supported(type) || ctx->fp32_matvec) return 0;
    const BlockGeom g = block_geom(type);
    if (k % g.elems || (static_cast<uint64_t>(k) / g.elems * g.bytes) % 16) return 0;
    return gemv_mma_norm_ok(type, k, m, ctx->dev) ? 1 : 0;
}

// ---- dense FFN fusions: SwiGLU in the gate/up launch, residual add in the down launch ----
// (the reference's dense builder issues gate, up, dispatch_silu_mul, down and an optional
// elementwise_add of the residual: src/inference/models/qwen35/gpu_ffn.rs:896-960)

HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu_supported(hf2q_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t type, uint32_t x_dtype) {
    if (!ctx || !type_supported(type) || n == 0 || k == 0 || ctx->fp32_matvec) return 0;
    const BlockGeom g = block_geom(type);
    if (k % g.elems || (static_cast<uint64_t>(k) / g.elems * g.bytes) % 16) return 0;
    return gemv_mma_swiglu_ok(type, k, m, x_dtype, ctx->dev) ? 1 : 0;
}

static int32_t swiglu_impl(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate, const void* w_up, float* y,
                           uint32_t m, uint32_t n, uint32_t k, uint32_t type, const float* norm_w, float norm_eps) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w_gate || !w_up || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_swiglu: null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_swiglu: x_dtype %u (want F32 or BF16)", x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, "qmatmul_swiglu");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    GemvArgs a{};
    a.w = w_gate; a.w2 = w_up; a.x = x; a.y = y;
    a.x_dtype = x_dtype; a.type = type;
    a.m = m; a.n = n; a.k = k;
    a.slots = 1; a.top_k = 1; a.n_experts = 0;
    a.swiglu = true;
    a.status = ctx->status;
    a.norm_weight = norm_w;
    a.norm_eps = norm_eps;
    GemvArgs up = a;
    up.w = w_up;
    if (norm_w && (x_dtype != HF2Q_DT_F32 || !gemv_mma_norm_ok(type, k, m, ctx->dev)))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "norm_qmatmul_swiglu: the fused RMSNorm takes 1..4 f32 rows of k <= 4096 (m=%u, k=%u)", m, k);
    if (!hf2q_cuda_qmatmul_swiglu_supported(ctx, m, n, k, type, x_dtype) || !gemv_mma_supported(a) || !gemv_mma_supported(up))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT,
                    "qmatmul_swiglu: m=%u k=%u does not fit one fused launch (ask hf2q_cuda_qmatmul_swiglu_supported; needs 16-byte aligned rows, "
                    "k %% 256 == 0, k > 1024 and all activations resident)", m, k);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_gemv_mma(a, ctx->dev, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_swiglu launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate,
                                          const void* w_up, float* y, uint32_t m, uint32_t n, uint32_t k, uint32_t type) {
    return swiglu_impl(ctx, stream, x, x_dtype, w_gate, w_up, y, m, n, k, type, nullptr, 0.f);
}

HF2Q_API int32_t hf2q_cuda_norm_qmatmul_swiglu(hf2q_ctx* ctx, void* stream, const float* x, const float* norm_weight, float eps,
                                               const void* w_gate, const void* w_up, float* y, uint32_t m, uint32_t n, uint32_t k,
                                               uint32_t type) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!norm_weight) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "norm_qmatmul_swiglu: null norm weight");
    return swiglu_impl(ctx, stream, x, HF2Q_DT_F32, w_gate, w_up, y, m, n, k, type, norm_weight, eps);
}

HF2Q_API int32_t hf2q_cuda_qmatmul_add_supported(hf2q_ctx* ctx, uint32_t n, uint32_t k, uint32_t type, uint32_t x_dtype) {
    if (!ctx || !type_supported(type) || n == 0 || k == 0 || ctx->fp32_matvec) return 0;
    const BlockGeom g = block_geom(type);
    if (k % 256 || (static_cast<uint64_t>(k) / g.elems * g.bytes) % 16) return 0;
    return gemv_mma_max_rows(type, k, x_dtype, ctx->dev) > 0 ? 1 : 0;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_add(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w,
                                       const float* residual, float* y, uint32_t m, uint32_t n, uint32_t k, uint32_t type) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w || !y || !residual) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_add: null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_add: x_dtype %u (want F32 or BF16)", x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, "qmatmul_add");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    if (reinterpret_cast<uintptr_t>(residual) % 4 || reinterpret_cast<uintptr_t>(y) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_add: misaligned buffer");
    GemvArgs a{};
    a.w = w; a.x = x; a.y = y;
    a.x_dtype = x_dtype; a.type = type;
    a.n = n; a.k = k;
    a.slots = 1; a.top_k = 1; a.n_experts = 0;
    a.status = ctx->status;
    a.residual = residual;
    if (ctx->fp32_matvec || !gemv_mma_supported(a) || gemv_mma_max_rows(type, k, x_dtype, ctx->dev) == 0)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_add: needs the warp-MMA mat-vec (16-byte aligned rows, k %% 256 == 0)");
    DeviceGuard dg(ctx->device);
    return run_matvec(ctx, static_cast<cudaStream_t>(stream), a, m, "qmatmul_add launch");
}

// ---- the same two fusions for any number of activation rows: mat-vec kernels up to 8 rows, above that the
// tensor-core GEMM with the SwiGLU pair in one tile / the residual in the epilogue (workspace as for hf2q_cuda_qmatmul)

HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu_ws_supported(hf2q_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t type, uint32_t x_dtype) {
    if (!ctx || !type_supported(type) || n == 0 || k == 0 || m == 0 || ctx->fp32_matvec) return 0;
    if (m <= 8) return hf2q_cuda_qmatmul_swiglu_supported(ctx, m, n, k, type, x_dtype);
    const BlockGeom g = block_geom(type);
    if (k % 256 || (static_cast<uint64_t>(k) / g.elems * g.bytes) % 16) return 0;
    return gemm_tc_swiglu_supported(type) ? 1 : 0;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_swiglu_ws(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate,
                                             const void* w_up, float* y, uint32_t m, uint32_t n, uint32_t k, uint32_t type,
                                             void* workspace, uint64_t workspace_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (m <= 8) return swiglu_impl(ctx, stream, x, x_dtype, w_gate, w_up, y, m, n, k, type, nullptr, 0.f);
    const char* who = "qmatmul_swiglu_ws";
    if (!x || !w_gate || !w_up || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: x_dtype %u (want F32 or BF16)", who, x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, who);
    if (rc) return rc;
    if (reinterpret_cast<uintptr_t>(x) % dtype_size(x_dtype) || reinterpret_cast<uintptr_t>(y) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: misaligned buffer", who);
    if (ctx->fp32_matvec || !gemm_tc_swiglu_supported(type) || !gemm_tc_supported(type, w_gate, n, k) || !gemm_tc_supported(type, w_up, n, k))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: needs one of the five main formats, 16-byte aligned rows and k %% 256 == 0 "
                    "(ask hf2q_cuda_qmatmul_swiglu_ws_supported)", who);
    const uint64_t need = gemm_tc_workspace_bytes(m, k);
    if (!workspace || workspace_bytes < need)
        return fail(ctx, HF2Q_ERR_WORKSPACE, "%s: m=%u needs a workspace of %llu bytes (got %llu)", who, m, (unsigned long long)need,
                    (unsigned long long)workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: workspace must be 256-byte aligned", who);
    DeviceGuard dg(ctx->device);
    int nl = 0;
    const cudaError_t e = launch_gemm_tc_swiglu(type, w_gate, w_up, x, x_dtype, y, m, n, k, workspace, ctx->status, ctx->dev.sm_count,
                                                static_cast<cudaStream_t>(stream), &nl);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_swiglu_ws launch");
    ctx->launches += nl;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_add_ws_supported(hf2q_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t type, uint32_t x_dtype) {
    if (!ctx || m == 0) return 0;
    if (m <= 8) return hf2q_cuda_qmatmul_add_supported(ctx, n, k, type, x_dtype);
    if (!type_supported(type) || n == 0 || k == 0 || ctx->fp32_matvec) return 0;
    const BlockGeom g = block_geom(type);
    return (k % 256 == 0 && (static_cast<uint64_t>(k) / g.elems * g.bytes) % 16 == 0) ? 1 : 0;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_add_ws(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w,
                                          const float* residual, float* y, uint32_t m, uint32_t n, uint32_t k, uint32_t type,
                                          void* workspace, uint64_t workspace_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (m <= 8) return hf2q_cuda_qmatmul_add(ctx, stream, x, x_dtype, w, residual, y, m, n, k, type);
    const char* who = "qmatmul_add_ws";
    if (!x || !w || !y || !residual) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: x_dtype %u (want F32 or BF16)", who, x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, who);
    if (rc) return rc;
    if (reinterpret_cast<uintptr_t>(x) % dtype_size(x_dtype) || reinterpret_cast<uintptr_t>(y) % 4 || reinterpret_cast<uintptr_t>(residual) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: misaligned buffer", who);
    if (ctx->fp32_matvec || !gemm_tc_supported(type, w, n, k))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: needs 16-byte aligned rows and k %% 256 == 0 (ask hf2q_cuda_qmatmul_add_ws_supported)", who);
    const uint64_t need = gemm_tc_workspace_bytes(m, k);
    if (!workspace || workspace_bytes < need)
        return fail(ctx, HF2Q_ERR_WORKSPACE, "%s: m=%u needs a workspace of %llu bytes (got %llu)", who, m, (unsigned long long)need,
                    (unsigned long long)workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: workspace must be 256-byte aligned", who);
    DeviceGuard dg(ctx->device);
    int nl = 0;
    const cudaError_t e = launch_gemm_tc(type, w, x, x_dtype, y, m, n, k, workspace, ctx->status, ctx->dev.sm_count,
                                         static_cast<cudaStream_t>(stream), &nl, 0, false, residual);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_add_ws launch");
    ctx->launches += nl;
    return HF2Q_OK;
}

// ---- row-sharded mat-vec with the all-gather in its epilogue (several GPUs, one process each) ----

HF2Q_API int32_t hf2q_cuda_ipc_alloc(hf2q_ctx* ctx, uint64_t bytes, void** dev, uint8_t* handle64) {
    if (!ctx || !dev || !handle64 || bytes == 0) return HF2Q_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    DeviceGuard g(ctx->device);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { if (p) cudaFree(p); return cuda_fail(ctx, e, "ipc_alloc"); }
    memcpy(handle64, &h, 64);
    *dev = p;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_ipc_open(hf2q_ctx* ctx, const uint8_t* handle64, void** dev) {
    if (!ctx || !dev || !handle64) return HF2Q_ERR_INVALID_ARGUMENT;
    DeviceGuard g(ctx->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "ipc_open (peer access between the two GPUs is required)");
    *dev = p;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_ipc_close(hf2q_ctx* ctx, void* dev) {
    if (!ctx || !dev) return HF2Q_ERR_INVALID_ARGUMENT;
    DeviceGuard g(ctx->device);
    const cudaError_t e = cudaIpcCloseMemHandle(dev);
    return e == cudaSuccess ? HF2Q_OK : cuda_fail(ctx, e, "ipc_close");
}

HF2Q_API int32_t hf2q_cuda_qmatmul_gather(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w,
                                          const hf2q_gather* g, uint32_t m, uint32_t n, uint32_t k, uint32_t type) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w || !g) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: x_dtype %u", x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, "qmatmul_gather");
    if (rc) return rc;
    if (g->n_ranks < 1 || g->n_ranks > 8 || g->rank >= g->n_ranks || static_cast<uint64_t>(g->col0) + n > g->n_total)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: rank %u of %u, columns [%u, %u) of %u", g->rank, g->n_ranks, g->col0, g->col0 + n, g->n_total);
    for (uint32_t r = 0; r < g->n_ranks; ++r)
        if (!g->y_all[r] || !g->flags[r] || reinterpret_cast<uintptr_t>(g->y_all[r]) % 4 || reinterpret_cast<uintptr_t>(g->flags[r]) % 4)
            return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: buffer of rank %u missing or misaligned", r);
    {
        // every rank derives the others' arrival counts from n_rows[]: they must describe real shards
        uint64_t sum = 0;
        for (uint32_t r = 0; r < g->n_ranks; ++r) {
            if (g->n_rows[r] == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: n_rows[%u] is zero", r);
            sum += g->n_rows[r];
        }
        if (g->n_rows[g->rank] != n || sum > g->n_total)
            return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: n_rows[] (sum %llu, own %u) does not match n=%u, n_total=%u",
                        (unsigned long long)sum, g->n_rows[g->rank], n, g->n_total);
    }
    if (m == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    GemvArgs a{};
    a.w = w; a.x = x; a.y = static_cast<float*>(g->y_all[g->rank]);
    a.x_dtype = x_dtype; a.type = type;
    a.m = m; a.n = n; a.k = k;
    a.slots = 1; a.top_k = 1; a.n_experts = 0;
    a.status = ctx->status;
    // one launch only: every launch bumps the peers' counters once
    if (m > 8 || ctx->fp32_matvec || !gemv_mma_supported(a) || gemv_mma_max_rows(type, k, x_dtype, ctx->dev) < m)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather: needs m <= %u activation rows, 16-byte aligned weight rows and k %% 256 == 0",
                    gemv_mma_supported(a) ? gemv_mma_max_rows(type, k, x_dtype, ctx->dev) : 8u);
    GatherArgs ga{};
    for (uint32_t r = 0; r < g->n_ranks; ++r) { ga.y_all[r] = static_cast<float*>(g->y_all[r]); ga.flags[r] = static_cast<uint32_t*>(g->flags[r]); }
    ga.n_ranks = g->n_ranks; ga.rank = g->rank; ga.n_total = g->n_total; ga.col0 = g->col0;
    ga.wait_expected = g->wait_previous;
    for (uint32_t r = 0; r < g->n_ranks; ++r) ga.peer_ctas[r] = gemv_mma_grid_x(g->n_rows[r], k, ctx->dev);
    ga.wait_limit = ctx->wait_limit;
    a.gather = &ga;
    const cudaError_t e = launch_gemv_mma(a, ctx->dev, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_gather launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_gather_wait(hf2q_ctx* ctx, void* stream, const hf2q_gather* g) {
    if (!ctx || !g) return HF2Q_ERR_INVALID_ARGUMENT;
    if (g->n_ranks < 1 || g->n_ranks > 8 || g->rank >= g->n_ranks || !g->flags[g->rank])
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_wait: rank %u of %u", g->rank, g->n_ranks);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_gather_wait(static_cast<const uint32_t*>(g->flags[g->rank]), g->n_ranks, g->rank, ctx->wait_limit, ctx->status,
                                             static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "gather_wait launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_gather_supported(hf2q_ctx* ctx, const void* w, uint32_t m, uint32_t n, uint32_t k, uint32_t type, uint32_t x_dtype) {
    if (!ctx || !w || !type_supported(type) || m == 0 || m > 8 || n == 0 || k == 0 || ctx->fp32_matvec) return 0;
    GemvArgs a{};
    a.w = w; a.x = nullptr; a.x_dtype = x_dtype; a.type = type; a.m = m; a.n = n; a.k = k; a.slots = 1; a.top_k = 1;
    return gemv_mma_supported(a) && gemv_mma_max_rows(type, k, x_dtype, ctx->dev) >= m ? 1 : 0;
}

HF2Q_API int32_t hf2q_cuda_gather_copy(hf2q_ctx* ctx, void* stream, const hf2q_gather* g, const float* src, uint32_t n) {
    if (!ctx || !g) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!src || n == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_copy: null or empty source");
    if (g->n_ranks < 1 || g->n_ranks > 8 || g->rank >= g->n_ranks || static_cast<uint64_t>(g->col0) + n > g->n_total || g->n_rows[g->rank] != n)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_copy: rank %u of %u, columns [%u, %u) of %u, n_rows[rank]=%u", g->rank, g->n_ranks,
                    g->col0, g->col0 + n, g->n_total, g->n_rows[g->rank]);
    GatherArgs ga{};
    for (uint32_t r = 0; r < g->n_ranks; ++r) {
        if (!g->y_all[r] || !g->flags[r] || g->n_rows[r] == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_copy: buffer or n_rows of rank %u missing", r);
        ga.y_all[r] = static_cast<float*>(g->y_all[r]);
        ga.flags[r] = static_cast<uint32_t*>(g->flags[r]);
    }
    ga.n_ranks = g->n_ranks; ga.rank = g->rank; ga.n_total = g->n_total; ga.col0 = g->col0;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_gather_copy(src, ga, n, g->n_rows, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "gather_copy launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_gather_sum(hf2q_ctx* ctx, void* stream, const hf2q_gather* g, float* x, uint32_t n, uint32_t n_parts) {
    if (!ctx || !g) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || n == 0 || n_parts == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_sum: null or empty x");
    if (g->n_ranks < 1 || g->n_ranks > 8 || g->rank >= g->n_ranks || !g->flags[g->rank] || !g->y_all[g->rank])
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_sum: rank %u of %u", g->rank, g->n_ranks);
    if (static_cast<uint64_t>(n) * n_parts > g->n_total)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "gather_sum: %u parts x %u values exceed the buffer's %u columns", n_parts, n, g->n_total);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_gather_sum(static_cast<const uint32_t*>(g->flags[g->rank]), g->n_ranks, g->rank, ctx->wait_limit, ctx->status,
                                            static_cast<const float*>(g->y_all[g->rank]), n, n_parts, x, n, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "gather_sum launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_set_wait_limit(hf2q_ctx* ctx, uint64_t clock_ticks) {
    if (!ctx || clock_ticks == 0 || clock_ticks > (1ull << 40)) return HF2Q_ERR_INVALID_ARGUMENT;
    ctx->wait_limit = static_cast<long long>(clock_ticks);
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_static(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w,
                                          float* y, uint32_t m, uint32_t n, uint32_t k, uint32_t type) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_static: null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_static: x_dtype %u (want F32 or BF16)", x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, "qmatmul_static");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    if (reinterpret_cast<uintptr_t>(x) % dtype_size(x_dtype) || reinterpret_cast<uintptr_t>(y) % 4)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_static: misaligned buffer");
    if (!gemm_tc_supported(type, w, n, k))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_static: needs k %% 256 == 0 and 16-byte aligned weight rows (k=%u)", k);
    const uint64_t need = gemm_tc_workspace_bytes(m, k), have = gemm_tc_static_scratch_bytes();
    if (need > have)
        return fail(ctx, HF2Q_ERR_WORKSPACE, "qmatmul_static: m*k = %llu elements needs %llu bytes of scratch, the fixed array holds %llu (m*k <= %llu)",
                    (unsigned long long)m * k, (unsigned long long)need, (unsigned long long)have, (unsigned long long)(have / 2));
    DeviceGuard dg(ctx->device);
    void* scratch = nullptr;
    cudaError_t e = gemm_tc_static_scratch(ctx->device, &scratch);       // first call per device: cudaGetSymbolAddress
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_static: cudaGetSymbolAddress");
    int nl = 0;
    e = launch_gemm_tc(type, w, x, x_dtype, y, m, n, k, scratch, ctx->status, ctx->dev.sm_count, static_cast<cudaStream_t>(stream), &nl);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_static launch");
    ctx->launches += nl;
    return HF2Q_OK;
}

HF2Q_API uint64_t hf2q_cuda_qmatmul_static_max_elements(void) { return gemm_tc_static_scratch_bytes() / 2; }


HF2Q_API int32_t hf2q_cuda_qmatmul_host_async(hf2q_ctx* ctx, const void* x_host, uint32_t x_dtype, const void* w_dev,
                                              float* y_host, uint32_t m, uint32_t n, uint32_t k, uint32_t type) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x_host || !w_dev || !y_host) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_host: null pointer");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_host: x_dtype %u", x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, "qmatmul_host");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const size_t xb = static_cast<size_t>(m) * k * dtype_size(x_dtype), yb = static_cast<size_t>(m) * n * 4;
    hf2q_ctx::HostSlot& hs = ctx->hslot[ctx->hnext++ % hf2q_ctx::HOST_SLOTS];
    uint64_t wsb = 0;
    hf2q_cuda_qmatmul_workspace_bytes(m, n, k, type, x_dtype, &wsb);
    cudaError_t e = cudaSuccess;
    if (hs.x_bytes < xb || hs.y_bytes < yb || ctx->ws_bytes < wsb) {
        // growing a buffer frees the old one: nothing may still be using it
        e = cudaStreamSynchronize(ctx->in_stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->host_stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->out_stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host: sync before growing staging buffers");
        if ((rc = grow(ctx, &hs.x, &hs.x_bytes, xb, false))) return rc;
        if ((rc = grow(ctx, reinterpret_cast<void**>(&hs.y), &hs.y_bytes, yb, false))) return rc;
        if (wsb && (rc = grow(ctx, &ctx->ws, &ctx->ws_bytes, wsb, false))) return rc;
    }
    if (!hs.computed) {
        e = cudaEventCreateWithFlags(&hs.computed, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&hs.loaded, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&hs.drained, cudaEventDisableTiming);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host: event");
    }
    // copy-in: after the slot's previous kernel has read its activations
    if (hs.used) e = cudaStreamWaitEvent(ctx->in_stream, hs.computed, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(hs.x, x_host, xb, cudaMemcpyHostToDevice, ctx->in_stream);
    if (e == cudaSuccess) e = cudaEventRecord(hs.loaded, ctx->in_stream);
    // kernel: after the copy-in, and after the slot's previous copy-out has read its results
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->host_stream, hs.loaded, 0);
    if (e == cudaSuccess && hs.used) e = cudaStreamWaitEvent(ctx->host_stream, hs.drained, 0);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host: copy-in");
    rc = hf2q_cuda_qmatmul(ctx, ctx->host_stream, hs.x, x_dtype, w_dev, hs.y, m, n, k, type, ctx->ws, ctx->ws_bytes);
    if (rc) return rc;
    e = cudaEventRecord(hs.computed, ctx->host_stream);
    // copy-out
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->out_stream, hs.computed, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(y_host, hs.y, yb, cudaMemcpyDeviceToHost, ctx->out_stream);
    if (e == cudaSuccess) e = cudaEventRecord(hs.drained, ctx->out_stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host: copy-out");
    hs.used = true;
    return HF2Q_OK;
}

// Many host-buffer products in one call: the copies-in run ahead on their own stream, the kernels run back to back
// on one stream (so consecutive mat-vecs keep their programmatic-dependent-launch overlap), the copies-out follow
// group by group on a third stream.  One event pair per group of products instead of three event edges per product.
// A decode loop hands in the same batch again and again (same host buffers, same weights): the second time an
// unchanged batch arrives, the three streams' work is captured into one CUDA graph, and from then on the call is one
// graph launch.  Anything that changes (an item, a staging buffer that grew) falls back to plain enqueueing.
namespace {
// Group boundaries of a batch of n products: [b[g], b[g+1]) is group g.  Every boundary costs the two kernels around
// it their start-up overlap (~3 us); every product of the LAST group delays the end of the call by its copy-out
// (~7 us), and the first group's copies-in delay the start.  So: groups of 8 in the middle, tapering to single
// products at the end (.., 4, 4, 2, 2, 1, 1) and starting small (2, 4, ..).
std::vector<uint32_t> batch_groups(uint32_t n) {
    std::vector<uint32_t> head, mid, tail;
    uint32_t r = n;
    for (uint32_t s : {1u, 1u, 2u, 2u, 4u, 4u}) { if (r < s) break; tail.push_back(s); r -= s; }
    for (uint32_t s : {2u, 4u}) { if (r < s) break; head.push_back(s); r -= s; }
    while (r) { const uint32_t g = r < 8 ? r : 8; mid.push_back(g); r -= g; }
    std::vector<uint32_t> b{0};
    for (uint32_t s : head) b.push_back(b.back() + s);
    for (uint32_t s : mid) b.push_back(b.back() + s);
    for (auto it = tail.rbegin(); it != tail.rend(); ++it) b.push_back(b.back() + *it);
    return b;
}

uint64_t batch_key(const hf2q_ctx* ctx, const hf2q_host_product* items, uint32_t n_items) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](const void* p, size_t n) {
        const unsigned char* b = static_cast<const unsigned char*>(p);
        for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
    };
    for (uint32_t i = 0; i < n_items; ++i) {       // field by field: padding bytes of the struct are not data
        const hf2q_host_product& it = items[i];
        mix(&it.x_host, sizeof it.x_host); mix(&it.w_dev, sizeof it.w_dev); mix(&it.y_host, sizeof it.y_host);
        mix(&it.m, sizeof it.m); mix(&it.n, sizeof it.n); mix(&it.k, sizeof it.k);
        mix(&it.ggml_type, sizeof it.ggml_type); mix(&it.x_dtype, sizeof it.x_dtype);
    }
    mix(&ctx->bx, sizeof ctx->bx); mix(&ctx->by, sizeof ctx->by); mix(&ctx->ws, sizeof ctx->ws);
    return h ? h : 1;
}

// The row-sharded form of a batch: every product goes through the fused all-gather of `g` (buffer 0 of every rank in
// g->y_all[], buffer 1 buf_stride bytes behind it; product i uses buffer (first_buf + i) & 1), equal shards.
struct GatherBatch {
    const hf2q_gather* g;
    uint64_t buf_stride;
    uint32_t first_buf;
};

// Queues the batch on the three streams.  Returns HF2Q_OK or the first error (already recorded in the context).
int32_t batch_enqueue(hf2q_ctx* ctx, const hf2q_host_product* items, uint32_t n_items, const std::vector<size_t>& xo,
                      const std::vector<size_t>& yo, const GatherBatch* gb = nullptr) {
    cudaError_t e = cudaSuccess;
    uint8_t* bx = static_cast<uint8_t*>(ctx->bx);
    uint8_t* by = static_cast<uint8_t*>(ctx->by);
    const std::vector<uint32_t> bounds = batch_groups(n_items);
    for (uint32_t g = 0; g + 1 < bounds.size(); ++g) {
        const uint32_t i0 = bounds[g], i1 = bounds[g + 1];
        for (uint32_t i = i0; i < i1 && e == cudaSuccess; ++i)
            e = cudaMemcpyAsync(bx + xo[i], items[i].x_host, static_cast<size_t>(items[i].m) * items[i].k * dtype_size(items[i].x_dtype),
                                cudaMemcpyHostToDevice, ctx->in_stream);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->b_loaded[g], ctx->in_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->host_stream, ctx->b_loaded[g], 0);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: copy-in");
        for (uint32_t i = i0; i < i1; ++i) {
            const hf2q_host_product& it = items[i];
            if (it.m == 0) continue;
            if (!gb) {
                const int32_t rc = hf2q_cuda_qmatmul(ctx, ctx->host_stream, bx + xo[i], it.x_dtype, it.w_dev, reinterpret_cast<float*>(by + yo[i]), it.m,
                                                     it.n, it.k, it.ggml_type, ctx->ws, ctx->ws_bytes);
                if (rc) return rc;
                continue;
            }
            // the sharded product: columns [rank * n, (rank + 1) * n) of this product's buffer on every rank
            hf2q_gather gi = *gb->g;
            const uint64_t shift = ((gb->first_buf + i) & 1u) * gb->buf_stride;
            for (uint32_t r = 0; r < gi.n_ranks; ++r) {
                gi.y_all[r] = static_cast<uint8_t*>(gi.y_all[r]) + shift;
                gi.n_rows[r] = it.n;
            }
            gi.col0 = gi.rank * it.n;
            gi.wait_previous = 1;
            int32_t rc = hf2q_cuda_qmatmul_gather(ctx, ctx->host_stream, bx + xo[i], it.x_dtype, it.w_dev, &gi, it.m, it.n, it.k, it.ggml_type);
            if (rc) return rc;
            if (it.y_host) {
                // The full-width rows leave the gather buffer on the kernel stream, BEFORE this rank's next product is
                // queued: a peer stores product i+2 into this buffer once it has seen product i+1 from every rank.
                e = launch_gather_take(static_cast<const uint32_t*>(gi.flags[gi.rank]), gi.n_ranks, gi.rank, ctx->wait_limit, ctx->status,
                                       static_cast<const float*>(gi.y_all[gi.rank]), gi.n_total, gi.n_ranks * it.n, it.m,
                                       reinterpret_cast<float*>(by + yo[i]), ctx->dev.sm_count, ctx->host_stream);
                if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_gather_host_batch: copy out of the gather buffer");
                ctx->launches += 1;
            }
        }
        e = cudaEventRecord(ctx->b_computed[g], ctx->host_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->out_stream, ctx->b_computed[g], 0);
        for (uint32_t i = i0; i < i1 && e == cudaSuccess; ++i)
            if (items[i].m && items[i].y_host)
                e = cudaMemcpyAsync(items[i].y_host, by + yo[i], static_cast<size_t>(items[i].m) * items[i].n * 4 * (gb ? gb->g->n_ranks : 1u),
                                    cudaMemcpyDeviceToHost, ctx->out_stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: copy-out");
    }
    return HF2Q_OK;
}

// Captures batch_enqueue into ctx->b_graph.  False (and no graph) when anything about the capture fails; the streams
// are left usable and the caller enqueues the batch the plain way.
bool batch_capture(hf2q_ctx* ctx, const hf2q_host_product* items, uint32_t n_items, const std::vector<size_t>& xo,
                   const std::vector<size_t>& yo, uint64_t key) {
    if (ctx->b_graph) { cudaGraphExecDestroy(ctx->b_graph); ctx->b_graph = nullptr; ctx->b_graph_key = 0; }
    if (!ctx->b_fork) {
        if (cudaEventCreateWithFlags(&ctx->b_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ctx->b_join_in, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ctx->b_join_out, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
    }
    if (cudaStreamBeginCapture(ctx->host_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); return false; }
    const uint64_t launches0 = ctx->launches;
    bool ok = cudaEventRecord(ctx->b_fork, ctx->host_stream) == cudaSuccess &&
              cudaStreamWaitEvent(ctx->in_stream, ctx->b_fork, 0) == cudaSuccess &&
              cudaStreamWaitEvent(ctx->out_stream, ctx->b_fork, 0) == cudaSuccess;
    if (ok) ok = batch_enqueue(ctx, items, n_items, xo, yo) == HF2Q_OK;
    if (ok) ok = cudaEventRecord(ctx->b_join_in, ctx->in_stream) == cudaSuccess &&
                 cudaEventRecord(ctx->b_join_out, ctx->out_stream) == cudaSuccess &&
                 cudaStreamWaitEvent(ctx->host_stream, ctx->b_join_in, 0) == cudaSuccess &&
                 cudaStreamWaitEvent(ctx->host_stream, ctx->b_join_out, 0) == cudaSuccess;
    cudaGraph_t graph = nullptr;
    const cudaError_t ec = cudaStreamEndCapture(ctx->host_stream, &graph);      // always: it ends the capture on all three streams
    const uint64_t launches = ctx->launches - launches0;
    ctx->launches = launches0;                                                  // nothing ran yet
    if (ok && ec == cudaSuccess && graph && cudaGraphInstantiate(&ctx->b_graph, graph, 0) == cudaSuccess) {
        ctx->b_graph_key = key;
        ctx->b_graph_launches = launches;
    } else {
        ctx->b_graph = nullptr;
        ok = false;
    }
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    if (!ok) ctx->err[0] = 0;              // the plain path reports its own errors
    return ok;
}
}  // namespace

static int32_t host_batch_impl(hf2q_ctx* ctx, const hf2q_host_product* items, uint32_t n_items, const GatherBatch* gb) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    const char* who = gb ? "qmatmul_gather_host_batch" : "qmatmul_host_batch";
    if (!items && n_items) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null item array", who);
    if (n_items == 0) return HF2Q_OK;
    const uint32_t wide = gb ? gb->g->n_ranks : 1u;          // a gathered result is n_ranks shards wide
    std::vector<size_t> xo(n_items), yo(n_items);
    size_t xt = 0, yt = 0;
    uint64_t wsb = 0;
    for (uint32_t i = 0; i < n_items; ++i) {
        const hf2q_host_product& it = items[i];
        if (!it.x_host || !it.w_dev || (!it.y_host && !gb)) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: item %u has a null pointer", who, i);
        if (it.x_dtype != HF2Q_DT_F32 && it.x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: item %u x_dtype %u", who, i, it.x_dtype);
        const int32_t rc = check_matmul_shape(ctx, it.ggml_type, it.n, it.k, who);
        if (rc) return rc;
        if (gb && static_cast<uint64_t>(wide) * it.n > gb->g->n_total)
            return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: item %u: %u shards of %u rows exceed the group's %u columns", who, i, wide, it.n, gb->g->n_total);
        xo[i] = xt; yo[i] = yt;
        xt += (static_cast<size_t>(it.m) * it.k * dtype_size(it.x_dtype) + 255) & ~static_cast<size_t>(255);
        if (it.y_host) yt += (static_cast<size_t>(it.m) * it.n * 4 * wide + 255) & ~static_cast<size_t>(255);
        uint64_t w1 = 0;
        if (!gb) hf2q_cuda_qmatmul_workspace_bytes(it.m, it.n, it.k, it.ggml_type, it.x_dtype, &w1);
        if (w1 > wsb) wsb = w1;
    }
    if (yt == 0) yt = 256;
    DeviceGuard dg(ctx->device);
    cudaError_t e = cudaSuccess;
    const uint32_t n_groups = static_cast<uint32_t>(batch_groups(n_items).size()) - 1;
    if (ctx->bx_bytes < xt || ctx->by_bytes < yt || ctx->ws_bytes < wsb) {
        e = cudaStreamSynchronize(ctx->in_stream);            // growing frees the old buffers: nothing may still use them
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->host_stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->out_stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: sync before growing staging buffers");
        int32_t rc;
        if ((rc = grow(ctx, &ctx->bx, &ctx->bx_bytes, xt, false))) return rc;
        if ((rc = grow(ctx, &ctx->by, &ctx->by_bytes, yt, false))) return rc;
        if (wsb && (rc = grow(ctx, &ctx->ws, &ctx->ws_bytes, wsb, false))) return rc;
    }
    while (ctx->b_loaded.size() < n_groups) {
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess || cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess)
            return cuda_fail(ctx, cudaGetLastError(), "qmatmul_host_batch: event");
        ctx->b_loaded.push_back(a);
        ctx->b_computed.push_back(b);
    }
    if (!ctx->b_all_computed) {
        e = cudaEventCreateWithFlags(&ctx->b_all_computed, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->b_all_drained, cudaEventDisableTiming);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: event");
    }
    // (the sharded form is always enqueued: its buffer parity and the peers' state are not part of a key)
    const uint64_t key = gb ? 0 : batch_key(ctx, items, n_items);
    static const bool graphs_off = [] { const char* v = getenv("HF2Q_HOST_BATCH_GRAPH"); return v && v[0] == '0'; }();
    if (!gb && !graphs_off && key != ctx->b_nograph_key && key == ctx->b_last_key && key != ctx->b_graph_key &&
        !batch_capture(ctx, items, n_items, xo, yo, key))
        ctx->b_nograph_key = key;          // do not try again on every call
    if (!gb) ctx->b_last_key = key;
    if (!gb && ctx->b_graph && key == ctx->b_graph_key) {
        // the graph starts after everything queued on the kernel stream; the previous batch's copies-out must have read
        // the y staging (its copies-in were waited for by its kernels)
        if (ctx->b_used) e = cudaStreamWaitEvent(ctx->host_stream, ctx->b_all_drained, 0);
        if (e == cudaSuccess) e = cudaGraphLaunch(ctx->b_graph, ctx->host_stream);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->b_all_computed, ctx->host_stream);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->b_all_drained, ctx->host_stream);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: graph launch");
        ctx->launches += ctx->b_graph_launches;
        ctx->b_used = true;
        return HF2Q_OK;
    }
    if (ctx->b_used) {
        // the previous batch: its kernels have read the x staging, its copies-out the y staging
        e = cudaStreamWaitEvent(ctx->in_stream, ctx->b_all_computed, 0);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->host_stream, ctx->b_all_drained, 0);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: ordering after the previous batch");
    }
    if (const int32_t rc = batch_enqueue(ctx, items, n_items, xo, yo, gb)) return rc;
    e = cudaEventRecord(ctx->b_all_computed, ctx->host_stream);
    if (e == cudaSuccess) e = cudaEventRecord(ctx->b_all_drained, ctx->out_stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_host_batch: events");
    ctx->b_used = true;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_host_batch(hf2q_ctx* ctx, const hf2q_host_product* items, uint32_t n_items) {
    return host_batch_impl(ctx, items, n_items, nullptr);
}

HF2Q_API int32_t hf2q_cuda_qmatmul_gather_host_batch(hf2q_ctx* ctx, const hf2q_gather* g, uint64_t buf_stride, uint32_t first_buf,
                                                     const hf2q_host_product* items, uint32_t n_items) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!g || g->n_ranks == 0 || g->n_ranks > 8 || g->rank >= g->n_ranks)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_gather_host_batch: bad group");
    const GatherBatch gb{g, buf_stride, first_buf & 1u};
    return host_batch_impl(ctx, items, n_items, &gb);
}

HF2Q_API int32_t hf2q_cuda_host_sync(hf2q_ctx* ctx) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    DeviceGuard dg(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->out_stream);      // every copy-out waited for its kernel, which waited for its copy-in
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->host_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->in_stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "host_sync");
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_host(hf2q_ctx* ctx, const void* x_host, uint32_t x_dtype, const void* w_dev,
                                        float* y_host, uint32_t m, uint32_t n, uint32_t k, uint32_t type) {
    const int32_t rc = hf2q_cuda_qmatmul_host_async(ctx, x_host, x_dtype, w_dev, y_host, m, n, k, type);
    return rc ? rc : hf2q_cuda_host_sync(ctx);
}

// routed rows above which the grouped tensor-core product is used (the reference's
// MM_ID_ROUTING_THRESHOLD settled on 32, docs/ADR-013-qwen35-inference.md:1097-1103)
static constexpr uint32_t MM_ID_ROUTING_THRESHOLD = 32;

HF2Q_API int32_t hf2q_cuda_qmatmul_id_scratch_bytes(uint32_t n_experts, uint32_t max_rows, uint32_t k,
                                                    uint32_t x_dtype, uint64_t* out) {
    (void)x_dtype;
    if (!out) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = max_rows > MM_ID_ROUTING_THRESHOLD ? moe_scratch_layout(n_experts, max_rows, k).total : 0;
    return HF2Q_OK;
}

namespace {
// mul_mat_id for one stacked expert tensor (w_b == nullptr) or for two of the same geometry that
// share x and ids (the gate and up projections of an MoE layer).
int32_t run_mul_mat_id(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_a, const void* w_b,
                       const uint32_t* ids, float* y_a, float* y_b, uint32_t n_tokens, uint32_t top_k, uint32_t n, uint32_t k,
                       uint32_t n_experts, uint64_t expert_stride, uint32_t type, void* scratch, uint64_t scratch_bytes,
                       const char* who) {
    if (!x || !w_a || !ids || !y_a || (w_b && !y_b)) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: x_dtype %u", who, x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, who);
    if (rc) return rc;
    if (top_k == 0 || n_experts == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: top_k=%u n_experts=%u must be non-zero", who, top_k, n_experts);
    uint64_t min_stride = 0;
    hf2q_cuda_expert_stride(type, n, k, &min_stride);
    if (expert_stride < min_stride) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: expert_stride %llu < one [n,k] matrix (%llu bytes)", who, (unsigned long long)expert_stride, (unsigned long long)min_stride);
    if (expert_stride % 2 || reinterpret_cast<uintptr_t>(w_a) % 2 || reinterpret_cast<uintptr_t>(w_b) % 2)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: weights must be 2-byte aligned", who);
    if (n_tokens == 0) return HF2Q_OK;
    const uint64_t rows = static_cast<uint64_t>(n_tokens) * top_k;
    DeviceGuard dg(ctx->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows > MM_ID_ROUTING_THRESHOLD && rows / 32 + n_experts <= 65535 && !ctx->fp32_matvec &&
        gemm_tc_grouped_supported(type, w_a, expert_stride, n_experts, k) &&
        (!w_b || gemm_tc_grouped_supported(type, w_b, expert_stride, n_experts, k)) && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
        // many rows: sort by expert on the device and gather activations ONCE, then one grouped
        // tensor-core launch per expert tensor
        const MoeScratch lay = moe_scratch_layout(n_experts, static_cast<uint32_t>(rows), k);
        if (!scratch || scratch_bytes < lay.total)
            return fail(ctx, HF2Q_ERR_WORKSPACE, "%s: %llu routed rows need %llu bytes of scratch (got %llu)", who,
                        (unsigned long long)rows, (unsigned long long)lay.total, (unsigned long long)scratch_bytes);
        if (reinterpret_cast<uintptr_t>(scratch) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: scratch must be 256-byte aligned", who);
        const uint32_t nt = moe_token_tile(static_cast<uint32_t>(rows), n_experts);
        cudaError_t e = launch_moe_prep(ids, static_cast<uint32_t>(rows), n_experts, top_k, nt, x, x_dtype, k, y_a, y_b, n, scratch, lay,
                                        ctx->status, ctx->dev.sm_count, st);
        if (e == cudaSuccess)
            e = launch_gemm_tc_grouped(type, w_a, expert_stride, n_experts, static_cast<uint32_t>(rows), y_a, n, k, nt, scratch, lay,
                                       ctx->status, st);
        if (e == cudaSuccess && w_b)
            e = launch_gemm_tc_grouped(type, w_b, expert_stride, n_experts, static_cast<uint32_t>(rows), y_b, n, k, nt, scratch, lay,
                                       ctx->status, st);
        if (e != cudaSuccess) return cuda_fail(ctx, e, who);
        ctx->launches += w_b ? 4 : 3;
        return HF2Q_OK;
    }
    // per-row mat-vec, at most 32768 routed rows per launch (grid.y limit is 65535); a pair shares the launch
    if (top_k > 16384) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: top_k=%u exceeds 16384", who, top_k);
    const uint64_t chunk = (w_b ? 16384 : 32768) / top_k * top_k;
    for (uint64_t r0 = 0; r0 < rows; ) {
        const uint64_t cnt = rows - r0 < chunk ? rows - r0 : chunk;
        GemvArgs a{};
        a.w = w_a;
        a.x = static_cast<const uint8_t*>(x) + (r0 / top_k) * k * dtype_size(x_dtype);
        a.y = y_a + r0 * n;
        a.ids = ids + r0;
        a.expert_stride = expert_stride;
        a.x_dtype = x_dtype;
        a.type = type;
        a.m = 1; a.n = n; a.k = k;
        a.slots = static_cast<uint32_t>(cnt);
        a.top_k = top_k;
        a.n_experts = n_experts;
        a.status = ctx->status;
        cudaError_t e;
        int nl = 1;
        if (!ctx->fp32_matvec && gemv_mma_supported(a) && gemv_mma_max_rows(type, k, x_dtype, ctx->dev) > 0) {
            if (w_b) { a.w2 = w_b; a.y2 = y_b + r0 * n; }
            e = launch_gemv_mma(a, ctx->dev, st);
        } else {
            e = launch_gemv(a, ctx->dev, st, &nl);
            if (e == cudaSuccess && w_b) {
                int nl2 = 1;
                a.w = w_b; a.y = y_b + r0 * n;
                e = launch_gemv(a, ctx->dev, st, &nl2);
                nl += nl2;
            }
        }
        if (e != cudaSuccess) return cuda_fail(ctx, e, who);
        ctx->launches += nl;
        r0 += cnt;
    }
    return HF2Q_OK;
}
}  // namespace

HF2Q_API int32_t hf2q_cuda_qmatmul_id(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                      const void* w_stacked, const uint32_t* ids, float* y, uint32_t n_tokens,
                                      uint32_t top_k, uint32_t n, uint32_t k, uint32_t n_experts,
                                      uint64_t expert_stride, uint32_t type, void* scratch, uint64_t scratch_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    return run_mul_mat_id(ctx, stream, x, x_dtype, w_stacked, nullptr, ids, y, nullptr, n_tokens, top_k, n, k, n_experts,
                          expert_stride, type, scratch, scratch_bytes, "qmatmul_id");
}

HF2Q_API int32_t hf2q_cuda_qmatmul_id_pair(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                           const void* w_a, const void* w_b, const uint32_t* ids, float* y_a, float* y_b,
                                           uint32_t n_tokens, uint32_t top_k, uint32_t n, uint32_t k, uint32_t n_experts,
                                           uint64_t expert_stride, uint32_t type, void* scratch, uint64_t scratch_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!w_b || !y_b) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "qmatmul_id_pair: null pointer");
    return run_mul_mat_id(ctx, stream, x, x_dtype, w_a, w_b, ids, y_a, y_b, n_tokens, top_k, n, k, n_experts, expert_stride, type,
                          scratch, scratch_bytes, "qmatmul_id_pair");
}

// gate and up of an MoE layer with the SwiGLU in the epilogue: few routed rows only (the mat-vec path)
HF2Q_API int32_t hf2q_cuda_qmatmul_id_swiglu_supported(hf2q_ctx* ctx, uint32_t n_tokens, uint32_t top_k, uint32_t n, uint32_t k,
                                                       uint32_t type, uint32_t x_dtype) {
    if (!ctx || !type_supported(type) || n == 0 || k == 0 || top_k == 0 || ctx->fp32_matvec) return 0;
    if (static_cast<uint64_t>(n_tokens) * top_k > MM_ID_ROUTING_THRESHOLD) return 0;
    const BlockGeom g = block_geom(type);
    if (k % g.elems || (static_cast<uint64_t>(k) / g.elems * g.bytes) % 16) return 0;
    return gemv_mma_swiglu_ok(type, k, 1, x_dtype, ctx->dev) ? 1 : 0;
}

HF2Q_API int32_t hf2q_cuda_qmatmul_id_swiglu(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype,
                                             const void* w_gate, const void* w_up, const uint32_t* ids, float* y,
                                             uint32_t n_tokens, uint32_t top_k, uint32_t n, uint32_t k, uint32_t n_experts,
                                             uint64_t expert_stride, uint32_t type) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    const char* who = "qmatmul_id_swiglu";
    if (!x || !w_gate || !w_up || !ids || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: x_dtype %u", who, x_dtype);
    int32_t rc = check_matmul_shape(ctx, type, n, k, who);
    if (rc) return rc;
    if (top_k == 0 || n_experts == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: top_k=%u n_experts=%u must be non-zero", who, top_k, n_experts);
    uint64_t min_stride = 0;
    hf2q_cuda_expert_stride(type, n, k, &min_stride);
    if (expert_stride < min_stride) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: expert_stride %llu < one [n,k] matrix (%llu bytes)", who, (unsigned long long)expert_stride, (unsigned long long)min_stride);
    if (n_tokens == 0) return HF2Q_OK;
    GemvArgs a{};
    a.w = w_gate; a.w2 = w_up; a.swiglu = true;
    a.x = x; a.y = y; a.ids = ids;
    a.expert_stride = expert_stride;
    a.x_dtype = x_dtype; a.type = type;
    a.m = 1; a.n = n; a.k = k;
    a.slots = n_tokens * top_k;
    a.top_k = top_k; a.n_experts = n_experts;
    a.status = ctx->status;
    GemvArgs up = a;
    up.w = w_up;
    if (!hf2q_cuda_qmatmul_id_swiglu_supported(ctx, n_tokens, top_k, n, k, type, x_dtype) || !gemv_mma_supported(a) || !gemv_mma_supported(up))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: %u routed rows of k=%u do not fit the fused launch (ask hf2q_cuda_qmatmul_id_swiglu_supported)",
                    who, n_tokens * top_k, k);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_gemv_mma(a, ctx->dev, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "qmatmul_id_swiglu launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

// ---- the routed experts of an MoE layer in four launches: sort + gather, gate/up pair with the SwiGLU in the
// epilogue writing the f16 activation panel in expert-sorted order, the down product reading that panel and
// scattering its rows back to routed-row order.  (The reference runs mul_mat_id, mul_mat_id, silu_mul,
// mul_mat_id: gpu_ffn.rs:2606-2760.)

HF2Q_API int32_t hf2q_cuda_moe_experts_scratch_bytes(uint32_t n_experts, uint32_t max_rows, uint32_t hidden, uint32_t ffn, uint64_t* out) {
    if (!out) return HF2Q_ERR_INVALID_ARGUMENT;
    const uint64_t act = (static_cast<uint64_t>(max_rows) * ffn * 2 + 255) & ~255ull;
    *out = moe_scratch_layout(n_experts, max_rows, hidden).total + act;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_moe_experts_supported(hf2q_ctx* ctx, uint32_t n_tokens, uint32_t top_k, uint32_t hidden, uint32_t ffn,
                                                 uint32_t n_experts, uint32_t type_gate_up, uint32_t type_down) {
    if (!ctx || ctx->fp32_matvec || !gemm_tc_swiglu_supported(type_gate_up) || !type_supported(type_down)) return 0;
    const uint64_t rows = static_cast<uint64_t>(n_tokens) * top_k;
    if (rows <= MM_ID_ROUTING_THRESHOLD || rows / 32 + n_experts > 65535 || n_experts == 0 || n_experts > 2048) return 0;
    const BlockGeom gg = block_geom(type_gate_up), gd = block_geom(type_down);
    if (hidden % 256 || ffn % 256) return 0;
    if ((static_cast<uint64_t>(hidden) / gg.elems * gg.bytes) % 16 || (static_cast<uint64_t>(ffn) / gd.elems * gd.bytes) % 16) return 0;
    return 1;
}

// route_w == nullptr: y = [n_tokens * top_k][hidden] rows of the routed slots.  Otherwise y = [n_tokens][hidden] and every
// slot's row is ADDED to its token's row, scaled by route_w[slot] (the caller has initialised y).
static int32_t moe_experts_impl(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate,
                                const void* w_up, const void* w_down, const uint32_t* ids, const float* route_w, float* y, uint32_t n_tokens,
                                uint32_t top_k, uint32_t hidden, uint32_t ffn, uint32_t n_experts, uint64_t stride_gate_up,
                                uint32_t type_gate_up, uint64_t stride_down, uint32_t type_down, void* scratch,
                                uint64_t scratch_bytes, const char* who) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !w_gate || !w_up || !w_down || !ids || !y) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: x_dtype %u", who, x_dtype);
    int32_t rc = check_matmul_shape(ctx, type_gate_up, ffn, hidden, who);
    if (!rc) rc = check_matmul_shape(ctx, type_down, hidden, ffn, who);
    if (rc) return rc;
    if (top_k == 0 || n_experts == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: top_k=%u n_experts=%u must be non-zero", who, top_k, n_experts);
    uint64_t min_gu = 0, min_d = 0;
    hf2q_cuda_expert_stride(type_gate_up, ffn, hidden, &min_gu);
    hf2q_cuda_expert_stride(type_down, hidden, ffn, &min_d);
    if (stride_gate_up < min_gu || stride_down < min_d)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: expert strides %llu / %llu are smaller than one matrix (%llu / %llu bytes)", who,
                    (unsigned long long)stride_gate_up, (unsigned long long)stride_down, (unsigned long long)min_gu, (unsigned long long)min_d);
    if (n_tokens == 0) return HF2Q_OK;
    if (!hf2q_cuda_moe_experts_supported(ctx, n_tokens, top_k, hidden, ffn, n_experts, type_gate_up, type_down) ||
        !gemm_tc_grouped_supported(type_gate_up, w_gate, stride_gate_up, n_experts, hidden) ||
        !gemm_tc_grouped_supported(type_gate_up, w_up, stride_gate_up, n_experts, hidden) ||
        !gemm_tc_grouped_supported(type_down, w_down, stride_down, n_experts, ffn) || reinterpret_cast<uintptr_t>(x) % 16)
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: %u x %u routed rows, hidden=%u, ffn=%u do not fit the grouped launches "
                    "(ask hf2q_cuda_moe_experts_supported; few rows take hf2q_cuda_qmatmul_id_swiglu + hf2q_cuda_qmatmul_id)", who,
                    n_tokens, top_k, hidden, ffn);
    const uint32_t rows = n_tokens * top_k;
    const MoeScratch lay = moe_scratch_layout(n_experts, rows, hidden);
    uint64_t need = 0;
    hf2q_cuda_moe_experts_scratch_bytes(n_experts, rows, hidden, ffn, &need);
    if (!scratch || scratch_bytes < need)
        return fail(ctx, HF2Q_ERR_WORKSPACE, "%s: %u routed rows need %llu bytes of scratch (got %llu)", who, rows, (unsigned long long)need,
                    (unsigned long long)scratch_bytes);
    if (reinterpret_cast<uintptr_t>(scratch) % 256) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: scratch must be 256-byte aligned", who);
    DeviceGuard dg(ctx->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* act16 = static_cast<uint8_t*>(scratch) + lay.total;
    const uint32_t nt = moe_token_tile(rows, n_experts);
    // the sort also zero-fills y: rows whose expert id is out of range stay zero, as in hf2q_cuda_qmatmul_id
    // (in the reducing form such rows simply add nothing)
    cudaError_t e = launch_moe_prep(ids, rows, n_experts, top_k, nt, x, x_dtype, hidden, route_w ? nullptr : y, nullptr, hidden, scratch, lay,
                                    ctx->status, ctx->dev.sm_count, st);
    if (e == cudaSuccess)
        e = launch_gemm_tc_grouped(type_gate_up, w_gate, stride_gate_up, n_experts, rows, nullptr, ffn, hidden, nt, scratch, lay, ctx->status,
                                   st, w_up, nullptr, act16);
    if (e == cudaSuccess)
        e = launch_gemm_tc_grouped(type_down, w_down, stride_down, n_experts, rows, y, hidden, ffn, nt, scratch, lay, ctx->status, st, nullptr,
                                   act16, nullptr, route_w, route_w ? y : nullptr, top_k);
    if (e != cudaSuccess) return cuda_fail(ctx, e, who);
    ctx->launches += 4;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_moe_experts(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate,
                                       const void* w_up, const void* w_down, const uint32_t* ids, float* y, uint32_t n_tokens,
                                       uint32_t top_k, uint32_t hidden, uint32_t ffn, uint32_t n_experts, uint64_t stride_gate_up,
                                       uint32_t type_gate_up, uint64_t stride_down, uint32_t type_down, void* scratch,
                                       uint64_t scratch_bytes) {
    return moe_experts_impl(ctx, stream, x, x_dtype, w_gate, w_up, w_down, ids, nullptr, y, n_tokens, top_k, hidden, ffn, n_experts,
                            stride_gate_up, type_gate_up, stride_down, type_down, scratch, scratch_bytes, "moe_experts");
}

HF2Q_API int32_t hf2q_cuda_moe_experts_reduce(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const void* w_gate,
                                              const void* w_up, const void* w_down, const uint32_t* ids, const float* weights, float* out,
                                              uint32_t n_tokens, uint32_t top_k, uint32_t hidden, uint32_t ffn, uint32_t n_experts,
                                              uint64_t stride_gate_up, uint32_t type_gate_up, uint64_t stride_down, uint32_t type_down,
                                              void* scratch, uint64_t scratch_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!weights) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_experts_reduce: null routing weights");
    return moe_experts_impl(ctx, stream, x, x_dtype, w_gate, w_up, w_down, ids, weights, out, n_tokens, top_k, hidden, ffn, n_experts,
                            stride_gate_up, type_gate_up, stride_down, type_down, scratch, scratch_bytes, "moe_experts_reduce");
}

HF2Q_API int32_t hf2q_cuda_moe_softmax_topk(hf2q_ctx* ctx, void* stream, const float* logits, uint32_t* ids,
                                            float* weights, uint32_t n_tokens, uint32_t n_experts, uint32_t top_k) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!logits || !ids || !weights) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_softmax_topk: null pointer");
    if (top_k == 0 || top_k > n_experts) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_softmax_topk: top_k=%u must be in 1..n_experts=%u", top_k, n_experts);
    if (n_experts > 3072) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_softmax_topk: n_experts=%u exceeds 3072", n_experts);
    if (n_tokens == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_softmax_topk(logits, ids, weights, n_tokens, n_experts, top_k, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "moe_softmax_topk launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_silu_mul(hf2q_ctx* ctx, void* stream, const float* gate, const float* up, float* out, uint64_t n) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!gate || !up || !out) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "silu_mul: null pointer");
    if (n == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_silu_mul(gate, up, out, n, ctx->dev.sm_count, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "silu_mul launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_moe_combine(hf2q_ctx* ctx, void* stream, const float* y, const float* weights, const float* shared,
                                       const float* shared_gate_logit, const float* residual, float* out, uint32_t n_tokens,
                                       uint32_t top_k, uint32_t hidden) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!out || (top_k && (!y || !weights))) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_combine: null pointer");
    if (hidden == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_combine: hidden must be non-zero");
    if (n_tokens == 0) return HF2Q_OK;
    if (n_tokens > 65535) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "moe_combine: n_tokens=%u exceeds 65535 per call", n_tokens);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_moe_combine(y, weights, shared, shared_gate_logit, residual, out, n_tokens, top_k, hidden,
                                             static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "moe_combine launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_router_logits(hf2q_ctx* ctx, void* stream, const void* x, uint32_t x_dtype, const float* router,
                                         float* logits, uint32_t n_tokens, uint32_t n_experts, uint32_t hidden) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !router || !logits || n_experts == 0 || hidden == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "router_logits: null pointer or empty shape");
    if (x_dtype != HF2Q_DT_F32 && x_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "router_logits: x_dtype %u (want F32 or BF16)", x_dtype);
    if (n_tokens == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_router_logits(x, x_dtype == HF2Q_DT_BF16, router, logits, n_tokens, n_experts, hidden, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "router_logits launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_rowdot(hf2q_ctx* ctx, void* stream, const float* x, const float* v, float* out, uint32_t n_tokens,
                                  uint32_t hidden) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !v || !out) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "rowdot: null pointer");
    if (n_tokens == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_rowdot(x, v, out, n_tokens, hidden, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "rowdot launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

// ---- the glue of a full decoder forward: embedding rows, RMSNorm, rotary + 8-bit KV append, attention, arg-max ----

namespace {
uint32_t attn_splits(const hf2q_ctx* ctx, uint32_t n_kv) {
    uint32_t s = n_kv ? static_cast<uint32_t>(2 * ctx->dev.sm_count) / n_kv : 1;
    return s < 1 ? 1 : s > 64 ? 64 : s;
}
int32_t check_kv(hf2q_ctx* ctx, const hf2q_kv_cache* kv, uint32_t n_q, const char* who) {
    if (!kv || !kv->k_codes || !kv->k_scale || !kv->v_codes || !kv->v_scale) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: null KV cache pointer", who);
    if (kv->head_dim != 128) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: head_dim %u (the attention kernels take 128)", who, kv->head_dim);
    const uint32_t g = kv->n_kv_heads ? n_q / kv->n_kv_heads : 0;
    if (kv->n_kv_heads == 0 || n_q % kv->n_kv_heads || !(g == 1 || g == 2 || g == 4 || g == 8))
        return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: %u query heads over %u KV heads (group size must be 1, 2, 4 or 8)", who, n_q, kv->n_kv_heads);
    if (kv->max_seq == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "%s: max_seq is zero", who);
    return HF2Q_OK;
}
KvCacheView view_of(const hf2q_kv_cache* kv) {
    return KvCacheView{static_cast<int8_t*>(kv->k_codes), static_cast<float*>(kv->k_scale), static_cast<int8_t*>(kv->v_codes),
                       static_cast<float*>(kv->v_scale), kv->max_seq};
}
}  // namespace

HF2Q_API int32_t hf2q_cuda_get_rows(hf2q_ctx* ctx, void* stream, const void* w, uint32_t type, uint32_t n_rows, uint32_t k,
                                    const uint32_t* ids, uint32_t m, float* out) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!w || !ids || !out) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "get_rows: null pointer");
    const int32_t rc = check_matmul_shape(ctx, type, n_rows, k, "get_rows");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    const BlockGeom g = block_geom(type);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_get_rows(type, w, static_cast<uint64_t>(k) / g.elems * g.bytes, n_rows, k, ids, m, out, ctx->status,
                                          static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "get_rows launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_rms_norm(hf2q_ctx* ctx, void* stream, float* x, const float* delta, const float* weight, float eps,
                                    void* out, uint32_t out_dtype, uint32_t m, uint32_t h) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !weight || !out || h == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "rms_norm: null pointer or h == 0");
    if (out_dtype != HF2Q_DT_F32 && out_dtype != HF2Q_DT_BF16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "rms_norm: out_dtype %u (want F32 or BF16)", out_dtype);
    if (m == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_rms_norm(x, delta, weight, eps, out, out_dtype, m, h, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "rms_norm launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_kv_cache_bytes(uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_seq, uint64_t* codes_bytes, uint64_t* scale_bytes) {
    if (!codes_bytes || !scale_bytes) return HF2Q_ERR_INVALID_ARGUMENT;
    *codes_bytes = static_cast<uint64_t>(n_kv_heads) * max_seq * head_dim;
    *scale_bytes = static_cast<uint64_t>(n_kv_heads) * max_seq * 4;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_rope_kv_append(hf2q_ctx* ctx, void* stream, float* qkv, uint32_t m, uint32_t n_q_heads, float theta,
                                          const uint32_t* pos, const hf2q_kv_cache* kv) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!qkv || !pos) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "rope_kv_append: null pointer");
    const int32_t rc = check_kv(ctx, kv, n_q_heads, "rope_kv_append");
    if (rc) return rc;
    if (m == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_rope_kv_append(qkv, m, n_q_heads, kv->n_kv_heads, kv->head_dim, pos, theta, view_of(kv), ctx->status,
                                                static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "rope_kv_append launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_attn_decode_scratch_bytes(hf2q_ctx* ctx, uint32_t n_q_heads, uint32_t n_kv_heads, uint64_t* out) {
    if (!ctx || !out || n_kv_heads == 0) return HF2Q_ERR_INVALID_ARGUMENT;
    *out = attn_decode_scratch_bytes(n_kv_heads, n_q_heads / n_kv_heads, attn_splits(ctx, n_kv_heads));
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_attn_decode(hf2q_ctx* ctx, void* stream, const float* q, uint32_t n_q_heads, const hf2q_kv_cache* kv,
                                       const uint32_t* pos, void* out, uint32_t out_dtype, void* scratch, uint64_t scratch_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!q || !pos || !out || !scratch) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "attn_decode: null pointer");
    const int32_t rc = check_kv(ctx, kv, n_q_heads, "attn_decode");
    if (rc) return rc;
    const uint32_t splits = attn_splits(ctx, kv->n_kv_heads);
    if (scratch_bytes < attn_decode_scratch_bytes(kv->n_kv_heads, n_q_heads / kv->n_kv_heads, splits))
        return fail(ctx, HF2Q_ERR_WORKSPACE, "attn_decode: scratch of %llu bytes is too small (ask hf2q_cuda_attn_decode_scratch_bytes)", (unsigned long long)scratch_bytes);
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_attn_decode(q, n_q_heads, kv->n_kv_heads, kv->head_dim, view_of(kv), pos, out, out_dtype,
                                             static_cast<float*>(scratch), splits, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "attn_decode launch");
    ctx->launches += 2;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_attn_decode_fused(hf2q_ctx* ctx, void* stream, const float* qkv, uint32_t n_q_heads, float theta,
                                             const hf2q_kv_cache* kv, const uint32_t* pos, void* out, uint32_t out_dtype, void* scratch,
                                             uint64_t scratch_bytes) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!qkv || !pos || !out || !scratch) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "attn_decode_fused: null pointer");
    const int32_t rc = check_kv(ctx, kv, n_q_heads, "attn_decode_fused");
    if (rc) return rc;
    const uint32_t splits = attn_splits(ctx, kv->n_kv_heads);
    if (scratch_bytes < attn_decode_scratch_bytes(kv->n_kv_heads, n_q_heads / kv->n_kv_heads, splits))
        return fail(ctx, HF2Q_ERR_WORKSPACE, "attn_decode_fused: scratch of %llu bytes is too small (ask hf2q_cuda_attn_decode_scratch_bytes)", (unsigned long long)scratch_bytes);
    if (reinterpret_cast<uintptr_t>(scratch) % 16) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "attn_decode_fused: scratch must be 16-byte aligned");
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_attn_decode_fused(qkv, n_q_heads, kv->n_kv_heads, kv->head_dim, theta, view_of(kv), pos, out, out_dtype,
                                                   static_cast<float*>(scratch), splits, ctx->status, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "attn_decode_fused launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_attn_prefill(hf2q_ctx* ctx, void* stream, const float* qkv, uint32_t m, uint32_t n_q_heads,
                                        const hf2q_kv_cache* kv, uint32_t pos0, void* out, uint32_t out_dtype) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!qkv || !out) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "attn_prefill: null pointer");
    const int32_t rc = check_kv(ctx, kv, n_q_heads, "attn_prefill");
    if (rc) return rc;
    if (static_cast<uint64_t>(pos0) + m > kv->max_seq) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "attn_prefill: positions %u..%u exceed max_seq %u", pos0, pos0 + m, kv->max_seq);
    if (m == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const uint32_t stride = (n_q_heads + 2 * kv->n_kv_heads) * kv->head_dim;
    const cudaError_t e = launch_attn_prefill(qkv, stride, m, n_q_heads, kv->n_kv_heads, kv->head_dim, view_of(kv), pos0, out, out_dtype,
                                              n_q_heads * kv->head_dim, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "attn_prefill launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_argmax(hf2q_ctx* ctx, void* stream, const float* logits, uint32_t n, uint32_t* out_id, uint32_t* pos) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!logits || !out_id || n == 0) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "argmax: null pointer or n == 0");
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_argmax(logits, n, out_id, pos, ctx->misc, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "argmax launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API int32_t hf2q_cuda_add(hf2q_ctx* ctx, void* stream, float* x, const float* delta, uint64_t n) {
    if (!ctx) return HF2Q_ERR_INVALID_ARGUMENT;
    if (!x || !delta) return fail(ctx, HF2Q_ERR_INVALID_ARGUMENT, "add: null pointer");
    if (n == 0) return HF2Q_OK;
    DeviceGuard dg(ctx->device);
    const cudaError_t e = launch_add(x, delta, n, ctx->dev.sm_count, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "add launch");
    ctx->launches += 1;
    return HF2Q_OK;
}

HF2Q_API uint64_t hf2q_cuda_launch_count(const hf2q_ctx* ctx) { return ctx ? ctx->launches : 0; }
HF2Q_API int32_t hf2q_cuda_sm_count(const hf2q_ctx* ctx) { return ctx ? ctx->dev.sm_count : 0; }

}  // extern "C"
