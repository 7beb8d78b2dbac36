// K1 (tensor-memory variant): dequant-fused mat-vec for 1..8 activation rows on tcgen05.
//
//   y[t, r] = sum_k x[t, k] * dequant(W)[r, k]
//
// Same call sites as k1_gemv_mma.cu (quantized_matmul_ggml with m <= 8:
// src/inference/models/qwen35/gpu_ffn.rs:1236-1306, src/serve/forward_mlx.rs:9960-9968).  The
// product is HBM-bound, so what matters is (a) the cheapest possible unpack per weight element and
// (b) enough CTAs to keep every SM streaming.  This kernel takes both from the prefill GEMM:
//
//   * thread = weight row.  A CTA owns 128 rows; each of 8 dequantiser warps reads its rows' raw
//     block bytes from shared memory (16-byte vectors, conflict-free pitch), unpacks them with
//     f16x2 arithmetic and stores the f16 operand straight into TENSOR MEMORY (tcgen05.st, row =
//     TMEM lane).  No cross-lane shuffles, no shared-memory round trip, no per-element FMA.
//   * tcgen05.mma.kind::f16, M = 128, N = 16, K = 16, A from TMEM, B = the activations (f16,
//     K-major, 128-byte swizzled) built in shared memory ONCE per CTA, for its whole k range,
//     directly from the caller's bf16 / f32 rows while the first weight copies are in flight
//     (f32 rows are split hi + lo over two MMA columns), D in TMEM.
//   * raw weights arrive by 2-D tensor copies (TMA) into a 2-stage ring, one 256-element K-block of
//     128 rows per stage; 4 A buffers of 64 elements each pipeline dequantisers against the MMA warp.
//   * k is split over a CLUSTER of S <= 8 CTAs so that 32..224 row tiles still occupy 148 SMs; the
//     partial accumulators are combined through distributed shared memory in a fixed order
//     (rank 0 adds ranks 1..S-1): deterministic, no atomics, no workspace.
//
// Weights are rounded to f16 after scaling (as in the prefill GEMM), so results agree with the f64
// product to ~3e-4 relative L2 (gate 1e-3), not to the ~1e-6 of the integer-code MMA kernel.
// Every mbarrier wait is bounded; no multicast; no peer-GPU memory.
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace hf2q {

using namespace tc;

namespace {

constexpr int TILE_N = 128;
constexpr int KB = 256;
constexpr int NT = 16;              // MMA N: activation columns
constexpr int RAW_STAGES = 2;
constexpr int DEQ_WARPS = 8;
constexpr int THREADS = (DEQ_WARPS + 2) * 32;
constexpr uint32_t TMEM_COLS = 256;             // A: 4 x 32 columns, D: 16 columns at +128

struct TParams {
    const void* x;
    float* y;
    uint32_t x_bf16, m, ncols;      // ncols = m (bf16) or 2m (f32 split)
    uint32_t n, k, nkb, splits;
    uint32_t boxw, blk_bytes;
    uint32_t tile_bytes;            // one 64-element activation tile: 1024 (<= 8 columns) or 2048
    uint32_t max_nloc;              // K-blocks of the busiest cluster rank (sizes the activation panel)
    uint32_t* status;
};

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// store into the shared memory of CTA `rank` of this cluster, at the address `local` has here
__device__ __forceinline__ void st_dsmem_f32(const float* local, uint32_t rank, float v) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(v) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// 32 activation values of one column -> f16, written as four 16-byte chunks of the 128B-swizzled
// K-major tile (row = column c, 8-row groups 1024 bytes apart).
__device__ __forceinline__ void build_x_half(uint8_t* tile, const TParams& p, uint32_t c, uint32_t hh, uint32_t kglob,
                                             bool& clipped) {
    uint32_t packed[16];
    if (c < p.ncols) {
        float v[32];
        if (p.x_bf16) {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.x) +
                                                              static_cast<size_t>(c) * p.k + kglob + 32 * hh);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 r = __ldg(src + i);
                const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[8 * i + 2 * j] = __uint_as_float(rr[j] << 16);
                    v[8 * i + 2 * j + 1] = __uint_as_float(rr[j] & 0xffff0000u);
                }
            }
        } else {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) +
                                                                static_cast<size_t>(c >> 1) * p.k + kglob + 32 * hh);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 r = __ldg(src + i);
                v[4 * i] = r.x; v[4 * i + 1] = r.y; v[4 * i + 2] = r.z; v[4 * i + 3] = r.w;
            }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float a = v[2 * i], b = v[2 * i + 1];
            clipped |= (fabsf(a) > 65504.0f) | (fabsf(b) > 65504.0f);
            a = fminf(fmaxf(a, -65504.0f), 65504.0f);
            b = fminf(fmaxf(b, -65504.0f), 65504.0f);
            __half ha = __float2half_rn(a), hb = __float2half_rn(b);
            if (!p.x_bf16 && (c & 1)) {          // lo part of the f32 split
                ha = __float2half_rn(a - __half2float(ha));
                hb = __float2half_rn(b - __half2float(hb));
            }
            packed[i] = static_cast<uint32_t>(__half_as_ushort(ha)) | (static_cast<uint32_t>(__half_as_ushort(hb)) << 16);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[i] = 0u;
    }
    uint8_t* rowp = tile + (c >> 3) * 1024 + (c & 7) * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t chunk = 4 * hh + i;
        *reinterpret_cast<uint4*>(rowp + ((chunk ^ (c & 7)) << 4)) =
            make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    }
}

template <uint32_t TYPE>
__global__ void __launch_bounds__(THREADS, 2)
gemv_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const TParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t raw_stage = TILE_N * p.boxw;
    uint8_t* raw = smem;                                         // RAW_STAGES x 128 x boxw
    float* part = reinterpret_cast<float*>(raw + RAW_STAGES * raw_stage);     // [splits][16][128] split-k partials (used in rank 0)
    uint64_t* bars = reinterpret_cast<uint64_t*>(part + p.splits * NT * TILE_N);
    uint64_t* raw_full = bars;                  // [RAW_STAGES]
    uint64_t* raw_empty = raw_full + RAW_STAGES;
    uint64_t* a_full = raw_empty + RAW_STAGES;  // [4]
    uint64_t* a_empty = a_full + 4;
    uint64_t* d_full = a_empty + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
    // activation panel: max_nloc x 4 tiles (+ one spare tile: with <= 8 columns the MMA's rows 8..15
    // read the following tile, whose values land in columns that are never stored)
    uint8_t* xs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row0 = blockIdx.x * TILE_N;
    const uint32_t z = blockIdx.z;                                    // == rank in the cluster
    const uint32_t kb0 = (z * p.nkb) / p.splits, kb1 = ((z + 1) * p.nkb) / p.splits;
    const uint32_t nloc = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], DEQ_WARPS); }
        for (int s = 0; s < 4; ++s) { mbar_init(&a_full[s], 4); mbar_init(&a_empty[s], 1); }
        mbar_init(d_full, 1);
        mbar_fence_init();
    }
    if (warp == DEQ_WARPS + 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base;
    const uint32_t tmem_d = tmem_base + 128;
    bool ok = true;

    auto issue_raw = [&](uint32_t kbl) -> bool {
        const uint32_t rs = kbl % RAW_STAGES;
        if (kbl >= RAW_STAGES && !mbar_wait_bounded(&raw_empty[rs], ((kbl / RAW_STAGES) - 1) & 1, p.status)) return false;
        mbar_arrive_expect_tx(&raw_full[rs], raw_stage);
        const uint32_t byte0 = ((kb0 + kbl) * p.blk_bytes) & ~15u;
        tma_2d(raw + rs * raw_stage, &tmap_w, static_cast<int>(byte0 >> 1), static_cast<int>(row0), &raw_full[rs]);
        return true;
    };
    // prologue: start the first weight copies, then everyone builds the f16 activation panel
    if (warp == DEQ_WARPS && lane == 0)
        for (uint32_t kbl = 0; kbl < nloc && kbl < RAW_STAGES; ++kbl) issue_raw(kbl);
    {
        bool clipped = false;
        const uint32_t rows = p.tile_bytes >> 7;                  // 8 or 16 columns per tile
        const uint32_t units = nloc * 4 * rows * 2;
        for (uint32_t u = threadIdx.x; u < units; u += THREADS) {
            const uint32_t hh = u & 1, c = (u >> 1) % rows, tile = (u >> 1) / rows;     // tile = kbl*4 + q
            build_x_half(xs + tile * p.tile_bytes, p, c, hh, (kb0 + (tile >> 2)) * KB + (tile & 3) * 64, clipped);
        }
        if (clipped) atomicOr(p.status, STATUS_X_CLIPPED);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // generic writes -> tensor-core reads
    }
    __syncthreads();

    if (warp == DEQ_WARPS) {
        // ------------------------------ producer: remaining TMA copies of raw weight blocks
        if (lane == 0)
            for (uint32_t kbl = RAW_STAGES; kbl < nloc && ok; ++kbl) ok = issue_raw(kbl);
    } else if (warp == DEQ_WARPS + 1) {
        // ------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC = (1u << 4) | (static_cast<uint32_t>(NT >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
            for (uint32_t kbl = 0; kbl < nloc && ok; ++kbl) {
                for (uint32_t q = 0; q < 4 && ok; ++q) {
                    ok = mbar_wait_bounded(&a_full[q], kbl & 1, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t bdesc = smem_desc_sw128(smem_u32(xs + (kbl * 4 + q) * p.tile_bytes));
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk)
                        umma_ts(tmem_d, tmem_a + q * 32 + kk * 8, bdesc + 2 * kk, IDESC, (kbl | q | kk) != 0 ? 1u : 0u);
                    tc_commit(&a_empty[q]);
                }
            }
            if (ok && nloc > 0) tc_commit(d_full);
        }
    } else {
        // ------------------------------ dequantisers: warps 0-3 quarters {0,1}, warps 4-7 quarters {2,3}
        const uint32_t grp = static_cast<uint32_t>(warp) >> 2, quad = warp & 3;
        const uint32_t r = quad * 32 + lane;
        const uint32_t lane_addr = (quad * 32u) << 16;
        for (uint32_t kbl = 0; kbl < nloc; ++kbl) {
            const uint32_t rs = kbl % RAW_STAGES;
            if (ok) ok = mbar_wait_bounded(&raw_full[rs], (kbl / RAW_STAGES) & 1, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t off = ((kb0 + kbl) * p.blk_bytes) & 15u;
            with_row_block<TYPE>(off, [&](auto rb) {
                rb.load(raw + rs * raw_stage + r * p.boxw, off);
                if constexpr (decltype(rb)::IN_REGS) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raw_empty[rs]);      // the stage's bytes are in registers now
                }
                // quarter indices must be compile-time constants (they index register arrays)
                auto do_quarter = [&](auto qc) {
                    constexpr uint32_t q = decltype(qc)::value;
                    if (ok && kbl >= 1) ok = mbar_wait_bounded(&a_empty[q], (kbl - 1) & 1, p.status);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) {
                        tc_fence_after();
                        uint32_t out[32];
                        rb.quarter(static_cast<int>(q), out);
                        tmem_st32(tmem_a + lane_addr + q * 32, out);
                        tmem_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&a_full[q]);
                    }
                };
                if (grp == 0) {
                    do_quarter(std::integral_constant<uint32_t, 0>{});
                    do_quarter(std::integral_constant<uint32_t, 1>{});
                } else {
                    do_quarter(std::integral_constant<uint32_t, 2>{});
                    do_quarter(std::integral_constant<uint32_t, 3>{});
                }
                if constexpr (!decltype(rb)::IN_REGS) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raw_empty[rs]);
                }
            });
            if (!ok) break;
        }
        // ------------------------------ epilogue (warps 0-3 hold the 128 accumulator lanes)
        if (warp < 4) {
            uint32_t v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0u;
            if (ok && nloc > 0) ok = mbar_wait_bounded(d_full, 0, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (ok && nloc > 0) {
                tc_fence_after();
                tmem_ld16(tmem_d + lane_addr, v);
                tmem_wait_ld();
            }
            if (p.splits > 1) {
                // every rank deposits its partial accumulators in rank 0's shared memory (slot z)
#pragma unroll
                for (int j = 0; j < 16; ++j) st_dsmem_f32(part + (z * NT + j) * TILE_N + r, 0, __uint_as_float(v[j]));
            } else {
                const uint32_t row = row0 + r;
                if (row < p.n && ok) {
                    if (p.x_bf16) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (static_cast<uint32_t>(j) < p.m) p.y[static_cast<size_t>(j) * p.n + row] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (static_cast<uint32_t>(j) < p.m)
                                p.y[static_cast<size_t>(j) * p.n + row] = __uint_as_float(v[2 * j]) + __uint_as_float(v[2 * j + 1]);
                    }
                }
            }
        }
    }
    if (p.splits > 1) {
        // combine the cluster's partial accumulators in rank order through distributed shared memory
        cluster_sync_all();
        if (z == 0 && warp < 4) {
            const uint32_t r = (warp & 3) * 32 + lane;
            const uint32_t row = row0 + r;
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = part[j * TILE_N + r];
            for (uint32_t rank = 1; rank < p.splits; ++rank) {       // fixed order: deterministic
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += part[(rank * NT + j) * TILE_N + r];
            }
            if (row < p.n) {
                if (p.x_bf16) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (static_cast<uint32_t>(j) < p.m) p.y[static_cast<size_t>(j) * p.n + row] = acc[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (static_cast<uint32_t>(j) < p.m) p.y[static_cast<size_t>(j) * p.n + row] = acc[2 * j] + acc[2 * j + 1];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == DEQ_WARPS + 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// k-split factor.  A CTA has a fixed cost (barrier and TMEM set-up, first copy latency, cluster
// barrier), so use the fewest splits that still give every SM a CTA, then nudge S by one if that
// evens out the CTAs-per-SM count.  S <= 8 (portable cluster size) and S <= number of K-blocks.
uint32_t choose_splits(uint32_t tiles, uint32_t nkb, int sms) {
    uint32_t s0 = (static_cast<uint32_t>(sms) + tiles - 1) / tiles;
    const uint32_t smax = nkb < 8 ? nkb : 8;
    if (s0 > smax) s0 = smax;
    if (s0 < 1) s0 = 1;
    auto eff = [&](uint32_t s) {
        const uint32_t pieces = tiles * s, per_sm = (pieces + sms - 1) / sms;
        return static_cast<double>(pieces) / (static_cast<double>(per_sm) * sms);
    };
    uint32_t best = s0;
    if (s0 + 1 <= smax && eff(s0 + 1) > eff(s0) + 0.08) best = s0 + 1;
    return best;
}

template <uint32_t TYPE>
cudaError_t launch_t(const CUtensorMap& tw, const TParams& p, cudaStream_t st) {
    auto kern = gemv_tc_kernel<TYPE>;
    size_t smem = 1024 + static_cast<size_t>(RAW_STAGES) * TILE_N * p.boxw + static_cast<size_t>(p.splits) * NT * TILE_N * 4 + 256 + 1024 +
                  (static_cast<size_t>(p.max_nloc) * 4 + 1) * p.tile_bytes;
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    if (smem < 80 * 1024) smem = 80 * 1024;       // at most two CTAs per SM: each holds 256 TMEM columns
    static std::mutex mu;
    static bool attr_set = false;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
            attr_set = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((p.n + TILE_N - 1) / TILE_N, 1, p.splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = p.splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, tw, p);
}

}  // namespace

bool gemv_tc_supported(const GemvArgs& a) {
    const BlockGeom g = block_geom(a.type);
    const uint64_t row_bytes = static_cast<uint64_t>(a.k) / g.elems * g.bytes;
    const uint32_t cols = a.x_dtype == HF2Q_DT_BF16 ? a.m : 2 * a.m;
    return a.ids == nullptr && encode_fn() != nullptr && a.k % KB == 0 && row_bytes % 16 == 0 &&
           cols <= NT && a.m <= 8 && reinterpret_cast<uintptr_t>(a.w) % 16 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0;
}

cudaError_t launch_gemv_tc(const GemvArgs& a, const DeviceInfo& dev, cudaStream_t st) {
    const BlockGeom g = block_geom(a.type);
    const uint64_t row_bytes = static_cast<uint64_t>(a.k) / g.elems * g.bytes;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    TParams p{};
    p.x = a.x; p.y = a.y;
    p.x_bf16 = a.x_dtype == HF2Q_DT_BF16;
    p.m = a.m;
    p.ncols = p.x_bf16 ? a.m : 2 * a.m;
    p.n = a.n; p.k = a.k;
    p.nkb = a.k / KB;
    p.boxw = tc_boxw(a.type);
    p.blk_bytes = KB / g.elems * g.bytes;
    p.status = a.status;
    p.splits = choose_splits((a.n + TILE_N - 1) / TILE_N, p.nkb, dev.sm_count);
    p.tile_bytes = p.ncols <= 8 ? 1024 : 2048;
    p.max_nloc = (p.nkb + p.splits - 1) / p.splits;
    alignas(64) CUtensorMap tw;
    cuuint64_t dims[2] = {row_bytes / 2, a.n};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {p.boxw / 2, TILE_N};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(a.w), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    switch (a.type) {
        case HF2Q_TYPE_Q4_0: return launch_t<HF2Q_TYPE_Q4_0>(tw, p, st);
        case HF2Q_TYPE_Q8_0: return launch_t<HF2Q_TYPE_Q8_0>(tw, p, st);
        case HF2Q_TYPE_Q4_K: return launch_t<HF2Q_TYPE_Q4_K>(tw, p, st);
        case HF2Q_TYPE_Q5_K: return launch_t<HF2Q_TYPE_Q5_K>(tw, p, st);
        case HF2Q_TYPE_Q6_K: return launch_t<HF2Q_TYPE_Q6_K>(tw, p, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace hf2q
