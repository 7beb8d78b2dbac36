// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of hf2q's GGUF block codec and of the scalar f32 reference math its tests use
// for the quantized-weight matmul path.  Only the test-suite, the smoke check and the benchmark's
// CPU-baseline leg may load this library; the CUDA library never links or calls it.
//
// What follows which reference file (paths are relative to the hf2q source tree):
//   nearest_int / make_qx_quants / make_qkx2_quants / make_qkx3_quants / make_qp_quants
//                                   src/quantize/ggml_quants/common.rs:23-518
//   Q4_0 quantizer                  src/quantize/ggml_quants/q4_0.rs:30-159
//   Q8_0 quantizer                  src/quantize/ggml_quants/q8_0.rs:31-72
//   Q4_K quantizer, 6-bit unpack    src/quantize/ggml_quants/q4_k.rs:50-337
//   Q5_K quantizer                  src/quantize/ggml_quants/q5_k.rs:58-366
//   Q6_K quantizer                  src/quantize/ggml_quants/q6_k.rs:40-221
//   block / type sizes, type ids    src/quantize/ggml_quants/ggml_type.rs:18-133
//   f16 round trip before quantize  src/convert/orchestrator.rs:536-550
//   load-time simple Q4_0 encoder   src/inference/models/qwen35/gpu_full_attn.rs:427-451
//   matmul_a_by_bt                  src/inference/models/qwen35/ffn.rs:38-50
//   softmax_topk_renorm_cpu         src/inference/models/qwen35/gpu_ffn.rs:1879-1924
//
// The reference has no dequantiser of its own (it delegates to the external mlx-native crate,
// version 0.9.1, which is not part of the source tree).  The dequantisers here are the exact
// inverse of the quantizers' re-encode step: each quantizer recomputes the integer codes from
// (x + dmin*m) / (d*sc) with the STORED f16 d/dmin and the PACKED sub-block scales
// (q4_k.rs:183-197, q5_k.rs:100-123, q6_k.rs:96-110, q4_0.rs:47-64, q8_0.rs:59-67), which fixes
// field packing, scale unpacking and the affine map.  The Q4_0 form is additionally the same as
// the reference's in-tree test helper (gpu_ffn.rs:3945-3962).
//
// Pinning: the quantizers are checked byte-for-byte against the reference's 20 golden fixture
// files for these five formats (tests/fixtures/ggml_quants/*).  Dequantised VALUES are not pinned
// by any reference test ("parity unpinned" for the numbers); they are pinned here only through
// the re-encode identity and through a second, independent numpy restatement.
//
// Floating point discipline: the reference (Rust) never contracts a*b+c unless it spells
// mul_add.  Build with -ffp-contract=off; every fmaf() below stands where the Rust says mul_add.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <algorithm>
#include <numeric>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr float GROUP_MAX_EPS = 1e-15f;  // common.rs:15
constexpr int QK_K = 256;
constexpr int K_SCALE_SIZE = 12;

// ---- IEEE binary16 <-> binary32 (round to nearest even), as half::f16 does -----------------
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

uint16_t f32_to_f16(float f) {
    const uint32_t x = f32_bits(f);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) {                       // inf / nan
        if (ax == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | 0x7e00u | ((ax >> 13) & 0x3ffu));   // quiet nan, payload kept
    }
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to >= 65520 -> inf
    if (ax < 0x33000001u) return (uint16_t)sign;               // <= 2^-25 -> +-0 (ties to even)
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    uint32_t shift, half_e;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); half_e = 0; }   // subnormal result
    else         { shift = 13;                          half_e = (uint32_t)(e + 15); }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    uint32_t out;
    if (half_e == 0) out = q;                       // q may reach 0x400 -> smallest normal, fine
    else out = ((half_e - 1) << 10) + q;            // q includes the implicit bit (0x400..0x800)
    return (uint16_t)(sign | out);
}

float f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    const uint32_t m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        float v = (float)m * 5.9604644775390625e-08f;  // m * 2^-24, exact
        return sign ? -v : v;
    }
    if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

// common.rs:23-28
inline int nearest_int(float fval) {
    float val = fval + 12582912.0f;
    int32_t i; std::memcpy(&i, &val, 4);
    return (i & 0x007fffff) - 0x00400000;
}

// Rust `f32 as i8`: truncate toward zero, saturate, NaN -> 0.
inline int8_t sat_i8(float v) {
    if (std::isnan(v)) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)(int)v;
}

inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// common.rs:61-168.  qw == nullptr stands for the empty slice.
float make_qx_quants(int n, int nmax, const float* x, int8_t* L, int rmse_type, const float* qw) {
    float max = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        float ax = std::fabs(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < GROUP_MAX_EPS) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.0f;
    }
    const float nmax_f = (float)nmax;
    float iscale = -nmax_f / max;
    if (rmse_type == 0) {
        for (int i = 0; i < n; ++i) {
            int li = nearest_int(iscale * x[i]);
            L[i] = (int8_t)(nmax + clampi(li, -nmax, nmax - 1));
        }
        return 1.0f / iscale;
    }
    bool return_early = false;
    if (rmse_type < 0) { rmse_type = -rmse_type; return_early = true; }
    auto weight = [&](int i) -> float {
        if (qw) return qw[i];
        if (rmse_type == 1) return x[i] * x[i];
        if (rmse_type == 2) return 1.0f;
        if (rmse_type == 3) return std::fabs(x[i]);
        return std::sqrt(std::fabs(x[i]));
    };
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        int li = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        L[i] = (int8_t)(li + nmax);
        float w = weight(i);
        sumlx = fmaf(w * x[i], (float)li, sumlx);
        suml2 = fmaf(w * (float)li, (float)li, suml2);
    }
    float scale = suml2 != 0.0f ? sumlx / suml2 : 0.0f;
    if (return_early) return suml2 > 0.0f ? 0.5f * (scale + 1.0f / iscale) : 1.0f / iscale;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(nmax_f + 0.1f * (float)is) / max;
        sumlx = 0.0f; suml2 = 0.0f;
        for (int i = 0; i < n; ++i) {
            int li = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
            float w = weight(i);
            sumlx = fmaf(w * x[i], (float)li, sumlx);
            suml2 = fmaf(w * (float)li, (float)li, suml2);
        }
        if (suml2 > 0.0f && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) {
                int li = nearest_int(iscale * x[i]);
                L[i] = (int8_t)(nmax + clampi(li, -nmax, nmax - 1));
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

// common.rs:174-288 (weights given) and :294-410 (weights optional, x*x fallback; `max <= min`).
// The two differ only in the weight source and the degenerate-range test, so one body serves both.
float make_qkx_quants(bool v3, int n, int nmax, const float* x, const float* weights, uint8_t* L,
                      float* the_min, uint8_t* Laux, float rmin, float rdelta, int nstep,
                      bool use_mad) {
    auto W = [&](int i) -> float { return weights ? weights[i] : x[i] * x[i]; };
    float min = x[0], max = x[0];
    float sum_w = W(0);
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        float w = W(i);
        sum_w += w;
        sum_x = fmaf(w, x[i], sum_x);
    }
    if (min > 0.0f) min = 0.0f;
    const bool degenerate = v3 ? (max <= min) : (max == min);
    if (degenerate) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        *the_min = -min;
        return 0.0f;
    }
    float iscale = (float)nmax / (max - min);
    float scale = 1.0f / iscale;
    float best_error = 0.0f;
    for (int i = 0; i < n; ++i) {
        int l = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
        L[i] = (uint8_t)l;
        float diff = fmaf(scale, (float)L[i], min) - x[i];
        diff = use_mad ? std::fabs(diff) : diff * diff;
        best_error = fmaf(W(i), diff, best_error);
    }
    if (nstep < 1) { *the_min = -min; return scale; }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (max - min);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; ++i) {
            int l = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
            Laux[i] = (uint8_t)l;
            float w = W(i);
            float lf = (float)l;
            sum_l = fmaf(w, lf, sum_l);
            sum_l2 = fmaf(w * lf, lf, sum_l2);
            sum_xl = fmaf(w * lf, x[i], sum_xl);
        }
        float D = fmaf(sum_w, sum_l2, -sum_l * sum_l);
        if (D > 0.0f) {
            float this_scale = fmaf(sum_w, sum_xl, -sum_x * sum_l) / D;
            float this_min = fmaf(sum_l2, sum_x, -sum_l * sum_xl) / D;
            if (this_min > 0.0f) { this_min = 0.0f; this_scale = sum_xl / sum_l2; }
            float cur_error = 0.0f;
            for (int i = 0; i < n; ++i) {
                float diff = fmaf(this_scale, (float)Laux[i], this_min) - x[i];
                diff = use_mad ? std::fabs(diff) : diff * diff;
                cur_error = fmaf(W(i), diff, cur_error);
            }
            if (cur_error < best_error) {
                for (int i = 0; i < n; ++i) L[i] = Laux[i];
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

// common.rs:415-518
float make_qp_quants(int n, int nmax, const float* x, uint8_t* L, const float* quant_weights) {
    float max = 0.0f;
    for (int i = 0; i < n; ++i) if (x[i] > max) max = x[i];
    if (max < GROUP_MAX_EPS) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.0f;
    }
    float iscale = (float)nmax / max;
    for (int i = 0; i < n; ++i) L[i] = (uint8_t)nearest_int(iscale * x[i]);
    float scale = 1.0f / iscale;
    float best_mse = 0.0f;
    for (int i = 0; i < n; ++i) {
        float diff = fmaf(scale, -(float)L[i], x[i]);
        float w = quant_weights[i];
        best_mse = fmaf(w * diff, diff, best_mse);
    }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        float iscale_is = (0.1f * (float)is + (float)nmax) / max;
        float scale_is = 1.0f / iscale_is;
        float mse = 0.0f;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale_is * x[i]);
            if (l > nmax) l = nmax;
            float diff = fmaf(scale_is, -(float)l, x[i]);
            float w = quant_weights[i];
            mse = fmaf(w * diff, diff, mse);
        }
        if (mse < best_mse) { best_mse = mse; iscale = iscale_is; }
    }
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        if (l > nmax) l = nmax;
        L[i] = (uint8_t)l;
        float w = quant_weights[i];
        sumlx = fmaf(w * x[i], (float)l, sumlx);
        suml2 = fmaf(w * (float)l, (float)l, suml2);
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            float w = quant_weights[i];
            float cur_l = (float)L[i];
            float slx = fmaf(w * x[i], -cur_l, sumlx);
            float sl2 = fmaf(w * cur_l, -cur_l, suml2);
            if (slx > 0.0f && sl2 > 0.0f) {
                int new_l = nearest_int(x[i] * sl2 / slx);
                if (new_l > nmax) new_l = nmax;
                if ((uint8_t)new_l != L[i]) {
                    slx = fmaf(w * x[i], (float)new_l, slx);
                    sl2 = fmaf(w * (float)new_l, (float)new_l, sl2);
                    if (slx * slx * suml2 > sumlx * sumlx * sl2) {
                        L[i] = (uint8_t)new_l;
                        sumlx = slx; suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (n_changed == 0) break;
    }
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

// q4_k.rs:329-337
inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// q4_k.rs:166-173 / q5_k.rs:75-85
inline void pack_scale_min_k4(int j, uint8_t* s, uint8_t ls, uint8_t lm) {
    if (j < 4) { s[j] = ls; s[j + 4] = lm; }
    else {
        s[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
        s[j - 4] |= (uint8_t)((ls >> 4) << 6);
        s[j] |= (uint8_t)((lm >> 4) << 6);
    }
}

inline void put_f16(uint8_t* p, uint16_t h) { p[0] = (uint8_t)(h & 0xff); p[1] = (uint8_t)(h >> 8); }
inline uint16_t get_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// ---- Q4_0 ------------------------------------------------------------------------------------
// q4_0.rs:30-67
void q4_0_row_ref(const float* src, int64_t n, uint8_t* out) {
    const int qk = 32;
    for (int64_t i = 0; i < n / qk; ++i) {
        const float* b = src + i * qk;
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < qk; ++j) {
            float v = b[j];
            if (amax < std::fabs(v)) { amax = std::fabs(v); max = v; }
        }
        float d = max / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint8_t* o = out + i * 18;
        put_f16(o, f32_to_f16(d));
        for (int j = 0; j < qk / 2; ++j) {
            float x0 = b[j] * id, x1 = b[qk / 2 + j] * id;
            uint8_t xi0 = (uint8_t)std::min<int8_t>(sat_i8(x0 + 8.5f), 15);
            uint8_t xi1 = (uint8_t)std::min<int8_t>(sat_i8(x1 + 8.5f), 15);
            o[2 + j] = (uint8_t)(xi0 | (xi1 << 4));
        }
    }
}

// q4_0.rs:71-105
void q4_0_row_impl(const float* x, const float* imatrix, int64_t n_per_row, uint8_t* out) {
    float weight[32]; int8_t L[32];
    float sum_x2 = 0.0f;
    for (int64_t j = 0; j < n_per_row; ++j) sum_x2 += x[j] * x[j];
    float sigma2 = sum_x2 / (float)n_per_row;
    for (int64_t ib = 0; ib < n_per_row / 32; ++ib) {
        const float* xb = x + 32 * ib; const float* qw = imatrix + 32 * ib;
        for (int j = 0; j < 32; ++j) weight[j] = qw[j] * std::sqrt(sigma2 + xb[j] * xb[j]);
        float d = make_qx_quants(32, 8, xb, L, 1, weight);
        uint8_t* o = out + ib * 18;
        put_f16(o, f32_to_f16(d));
        for (int j = 0; j < 16; ++j) o[2 + j] = (uint8_t)((uint8_t)L[j] | ((uint8_t)L[j + 16] << 4));
    }
}

// ---- the 32-element formats the reference's tensor_type_fallback targets (standard_policy.rs:128-192)
// Rust `f32 as u8`: truncate toward zero, saturate, NaN -> 0.
inline uint8_t sat_u8(float v) {
    if (std::isnan(v)) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 255.0f) return 255;
    return (uint8_t)(int)v;
}
inline void put_u32(uint8_t* p, uint32_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); p[2] = (uint8_t)(v >> 16); p[3] = (uint8_t)(v >> 24); }
inline uint32_t get_u32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

// weight[j] = qw[j] * sqrt(sigma2 + x[j]^2) with sigma2 = mean(x^2) over the row (q4_1.rs:119-137 and siblings)
inline float row_sigma2(const float* x, int64_t n) {
    float sum_x2 = 0.0f;
    for (int64_t j = 0; j < n; ++j) sum_x2 += x[j] * x[j];
    return sum_x2 / (float)n;
}

// q4_1.rs:79-113 (no imatrix) and :116-160 (imatrix, make_qkx3_quants)
void q4_1_row(const float* x, const float* imatrix, int64_t n, uint8_t* out) {
    const float sigma2 = imatrix ? row_sigma2(x, n) : 0.0f;
    for (int64_t i = 0; i < n / 32; ++i) {
        const float* b = x + 32 * i;
        uint8_t* o = out + 20 * i;
        if (!imatrix) {
            float mn = 3.40282347e+38f, mx = -3.40282347e+38f;
            for (int j = 0; j < 32; ++j) { if (b[j] < mn) mn = b[j]; if (b[j] > mx) mx = b[j]; }
            float d = (mx - mn) / 15.0f;
            float id = d != 0.0f ? 1.0f / d : 0.0f;
            put_f16(o, f32_to_f16(d));
            put_f16(o + 2, f32_to_f16(mn));
            for (int j = 0; j < 16; ++j) {
                float x0 = (b[j] - mn) * id, x1 = (b[16 + j] - mn) * id;
                uint8_t xi0 = (uint8_t)std::min<int8_t>(sat_i8(x0 + 0.5f), 15);
                uint8_t xi1 = (uint8_t)std::min<int8_t>(sat_i8(x1 + 0.5f), 15);
                o[4 + j] = (uint8_t)(xi0 | (xi1 << 4));
            }
        } else {
            float weight[32]; uint8_t L[32], Laux[32];
            const float* qw = imatrix + 32 * i;
            for (int j = 0; j < 32; ++j) weight[j] = qw[j] * std::sqrt(sigma2 + b[j] * b[j]);
            float min_neg = 0.0f;
            float d = make_qkx_quants(true, 32, 15, b, weight, L, &min_neg, Laux, -0.9f, 0.05f, 36, false);
            put_f16(o, f32_to_f16(d));
            put_f16(o + 2, f32_to_f16(-min_neg));
            for (int j = 0; j < 16; ++j) o[4 + j] = (uint8_t)(L[j] | (L[j + 16] << 4));
        }
    }
}

// q5_0.rs:67-112 (no imatrix) and :114-193 (imatrix, make_qx_quants with nmax 16)
void q5_0_row(const float* x, const float* imatrix, int64_t n, uint8_t* out) {
    const float sigma2 = imatrix ? row_sigma2(x, n) : 0.0f;
    for (int64_t i = 0; i < n / 32; ++i) {
        const float* b = x + 32 * i;
        uint8_t* o = out + 22 * i;
        uint8_t q[32];
        float d;
        if (!imatrix) {
            float amax = 0.0f, mx = 0.0f;
            for (int j = 0; j < 32; ++j) { float av = std::fabs(b[j]); if (amax < av) { amax = av; mx = b[j]; } }
            d = mx / -16.0f;
            float id = d != 0.0f ? 1.0f / d : 0.0f;
            for (int j = 0; j < 32; ++j) {
                float v = b[j] * id + 16.5f;
                int xi = std::isnan(v) ? 0 : (int)v;                 // `as i32`: truncation toward zero
                q[j] = (uint8_t)std::min(xi, 31);
            }
        } else {
            float weight[32]; int8_t L[32];
            const float* qw = imatrix + 32 * i;
            for (int j = 0; j < 32; ++j) weight[j] = qw[j] * std::sqrt(sigma2 + b[j] * b[j]);
            d = make_qx_quants(32, 16, b, L, 1, weight);
            for (int j = 0; j < 32; ++j) q[j] = (uint8_t)L[j];
        }
        put_f16(o, f32_to_f16(d));
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            o[6 + j] = (uint8_t)((q[j] & 0x0F) | ((q[j + 16] & 0x0F) << 4));
            qh |= (uint32_t)((q[j] & 0x10) >> 4) << j;
            qh |= (uint32_t)((q[j + 16] & 0x10) >> 4) << (j + 16);
        }
        put_u32(o + 2, qh);
    }
}

// q5_1.rs:40-88 (no imatrix) and :90-150 (imatrix, make_qkx3_quants with nmax 31)
void q5_1_row(const float* x, const float* imatrix, int64_t n, uint8_t* out) {
    const float sigma2 = imatrix ? row_sigma2(x, n) : 0.0f;
    for (int64_t i = 0; i < n / 32; ++i) {
        const float* b = x + 32 * i;
        uint8_t* o = out + 24 * i;
        uint8_t q[32];
        if (!imatrix) {
            float mn = 3.40282347e+38f, mx = -3.40282347e+38f;
            for (int j = 0; j < 32; ++j) { if (b[j] < mn) mn = b[j]; if (b[j] > mx) mx = b[j]; }
            float d = (mx - mn) / 31.0f;
            float id = d != 0.0f ? 1.0f / d : 0.0f;
            put_f16(o, f32_to_f16(d));
            put_f16(o + 2, f32_to_f16(mn));
            for (int j = 0; j < 32; ++j) q[j] = sat_u8((b[j] - mn) * id + 0.5f);
        } else {
            float weight[32]; uint8_t Laux[32];
            const float* qw = imatrix + 32 * i;
            for (int j = 0; j < 32; ++j) weight[j] = qw[j] * std::sqrt(sigma2 + b[j] * b[j]);
            float the_min = 0.0f;
            float d = make_qkx_quants(true, 32, 31, b, weight, q, &the_min, Laux, -0.9f, 0.05f, 36, false);
            put_f16(o, f32_to_f16(d));
            put_f16(o + 2, f32_to_f16(-the_min));
        }
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            o[8 + j] = (uint8_t)((q[j] & 0x0F) | ((q[j + 16] & 0x0F) << 4));
            qh |= (uint32_t)((q[j] & 0x10) >> 4) << j;
            qh |= (uint32_t)((q[j + 16] & 0x10) >> 4) << (j + 16);
        }
        put_u32(o + 4, qh);
    }
}

// iq4_nl.rs: the 16-entry non-linear codebook and the single-block search with ntry = 7
const int8_t KVALUES_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// common.rs:33-55
inline int best_index_int8(const int8_t* val, int n, float x) {
    if (x <= (float)val[0]) return 0;
    if (x >= (float)val[n - 1]) return n - 1;
    int ml = 0, mu = n - 1;
    while (mu - ml > 1) {
        int mav = (ml + mu) / 2;
        if (x < (float)val[mav]) mu = mav; else ml = mav;
    }
    return x - (float)val[mu - 1] < (float)val[mu] - x ? mu - 1 : mu;
}

void iq4_nl_block(const float* x, const float* qw, uint8_t* out) {
    const int ntry = 7;
    const int8_t* values = KVALUES_IQ4NL;
    float sigma2 = 0.0f;
    for (int j = 0; j < 32; ++j) sigma2 += x[j] * x[j];
    sigma2 *= 2.0f / 32.0f;
    float weight[32]; uint8_t L[32] = {0};
    for (int j = 0; j < 32; ++j) weight[j] = qw ? qw[j] * std::sqrt(sigma2 + x[j] * x[j]) : x[j] * x[j];
    float amax = 0.0f, mx = 0.0f;
    for (int j = 0; j < 32; ++j) { float ax = std::fabs(x[j]); if (ax > amax) { amax = ax; mx = x[j]; } }
    float scale0 = 0.0f;
    const bool all_zero = amax < GROUP_MAX_EPS;
    if (!all_zero) {
        float d = -mx / (float)values[0];          // ntry > 0
        float id = 1.0f / d;
        float sumqx = 0.0f, sumq2 = 0.0f;
        for (int j = 0; j < 32; ++j) {
            int l = best_index_int8(values, 16, id * x[j]);
            L[j] = (uint8_t)l;
            float q = (float)values[l], w = weight[j];
            sumqx += w * q * x[j];
            sumq2 += w * q * q;
        }
        d = sumq2 > 0.0f ? sumqx / sumq2 : 0.0f;
        float best = d * sumqx;
        for (int itry = -ntry; itry <= ntry; ++itry) {
            id = ((float)itry + (float)values[0]) / mx;
            float sqx = 0.0f, sq2 = 0.0f;
            for (int j = 0; j < 32; ++j) {
                int l = best_index_int8(values, 16, id * x[j]);
                float q = (float)values[l], w = weight[j];
                sqx += w * q * x[j];
                sq2 += w * q * q;
            }
            if (sq2 > 0.0f && sqx * sqx > best * sq2) { d = sqx / sq2; best = d * sqx; }
        }
        scale0 = d;
        id = scale0 != 0.0f ? 1.0f / scale0 : 0.0f;
        for (int j = 0; j < 32; ++j) L[j] = (uint8_t)best_index_int8(values, 16, id * x[j]);
    }
    put_f16(out, f32_to_f16(scale0));
    for (int j = 0; j < 16; ++j) out[2 + j] = (uint8_t)(L[j] | (L[16 + j] << 4));
}

// ---- Q8_0 ------------------------------------------------------------------------------------
// q8_0.rs:31-72.  Rust f32::round is half-away-from-zero == roundf.
void q8_0_blocks(const float* src, int64_t n, uint8_t* out) {
    for (int64_t bi = 0; bi < n / 32; ++bi) {
        const float* b = src + bi * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) { float a = std::fabs(b[j]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint8_t* o = out + bi * 34;
        put_f16(o, f32_to_f16(d));
        for (int j = 0; j < 32; ++j) o[2 + j] = (uint8_t)sat_i8(std::round(b[j] * id));
    }
}

// ---- Q4_K / Q5_K shared tail ----------------------------------------------------------------
// Second-stage re-encode with the stored f16 d/dmin and unpacked 6-bit scales
// (q4_k.rs:176-197, q5_k.rs:92-123); L holds the first-stage codes and keeps them where d == 0.
void k45_reencode(const float* xb, uint16_t d_h, uint16_t dmin_h, const uint8_t* scales, uint8_t* L,
                  int qmax) {
    float d_dq = f16_to_f32(d_h), dmin_dq = f16_to_f32(dmin_h);
    for (int j = 0; j < QK_K / 32; ++j) {
        uint8_t sc, m; get_scale_min_k4(j, scales, &sc, &m);
        float d = d_dq * (float)sc;
        if (d == 0.0f) continue;
        float dm = dmin_dq * (float)m;
        for (int ii = 0; ii < 32; ++ii) {
            int l = nearest_int((xb[32 * j + ii] + dm) / d);
            L[32 * j + ii] = (uint8_t)clampi(l, 0, qmax);
        }
    }
}

// q4_k.rs:199-215
void q4_k_emit(uint16_t d_h, uint16_t dmin_h, const uint8_t* scales, const uint8_t* L, uint8_t* o) {
    put_f16(o, d_h); put_f16(o + 2, dmin_h);
    std::memcpy(o + 4, scales, K_SCALE_SIZE);
    uint8_t* q = o + 16;
    for (int j = 0; j < QK_K; j += 64)
        for (int l = 0; l < 32; ++l) *q++ = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
}

// q5_k.rs:125-158
void q5_k_emit(uint16_t d_h, uint16_t dmin_h, const uint8_t* scales, const uint8_t* L, uint8_t* o) {
    put_f16(o, d_h); put_f16(o + 2, dmin_h);
    std::memcpy(o + 4, scales, K_SCALE_SIZE);
    uint8_t* qh = o + 16; uint8_t* ql = o + 48;
    std::memset(qh, 0, 32); std::memset(ql, 0, 128);
    uint8_t m1 = 1, m2 = 2;
    for (int chunk = 0; chunk < 4; ++chunk) {
        int n = chunk * 64;
        for (int j = 0; j < 32; ++j) {
            int l1 = L[n + j];
            if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
            int l2 = L[n + j + 32];
            if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
            ql[chunk * 32 + j] = (uint8_t)((uint8_t)l1 | ((uint8_t)l2 << 4));
        }
        m1 = (uint8_t)(m1 << 2); m2 = (uint8_t)(m2 << 2);
    }
}

// q4_k.rs:89-217 (nmax 15, rmin -1, rdelta .1, nstep 20) and q5_k.rs:162-239 (31, -.5, .1, 15)
void k45_row_ref(const float* x, int64_t n, uint8_t* out, bool is_q5) {
    const int nmax = is_q5 ? 31 : 15;
    const float rmin = is_q5 ? -0.5f : -1.0f;
    const int nstep = is_q5 ? 15 : 20;
    const int bb = is_q5 ? 176 : 144;
    uint8_t L[QK_K], Laux[32];
    float weights[32], mins[8], scales[8];
    for (int64_t i = 0; i < n / QK_K; ++i) {
        const float* xb = x + i * QK_K;
        float max_scale = 0.0f, max_min = 0.0f;
        std::memset(L, 0, sizeof L);
        for (int j = 0; j < 8; ++j) {
            const float* sub = xb + 32 * j;
            float sum_x2 = 0.0f;
            for (int l = 0; l < 32; ++l) sum_x2 = fmaf(sub[l], sub[l], sum_x2);
            float av_x = std::sqrt(sum_x2 / 32.0f);
            for (int l = 0; l < 32; ++l) weights[l] = av_x + std::fabs(sub[l]);
            scales[j] = make_qkx_quants(false, 32, nmax, sub, weights, L + 32 * j, &mins[j], Laux,
                                        rmin, 0.1f, nstep, false);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        uint8_t sp[K_SCALE_SIZE] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t ls = (uint8_t)nearest_int(inv_scale * scales[j]);
            uint8_t lm = (uint8_t)nearest_int(inv_min * mins[j]);
            if (ls > 63) ls = 63;
            if (lm > 63) lm = 63;
            pack_scale_min_k4(j, sp, ls, lm);
        }
        uint16_t d_h = f32_to_f16(max_scale / 63.0f), dmin_h = f32_to_f16(max_min / 63.0f);
        k45_reencode(xb, d_h, dmin_h, sp, L, nmax);
        if (is_q5) q5_k_emit(d_h, dmin_h, sp, L, out + i * bb);
        else       q4_k_emit(d_h, dmin_h, sp, L, out + i * bb);
    }
}

// q4_k.rs:220-325 and q5_k.rs:242-312 (imatrix path; quant_weights spans the row)
void k45_row_impl(const float* x, const float* quant_weights, int64_t n, uint8_t* out, bool is_q5) {
    const int nmax = is_q5 ? 31 : 15;
    const int bb = is_q5 ? 176 : 144;
    uint8_t L[QK_K], Laux[32], Ls[8], Lm[8];
    float weights[32], sw[8], mins[8], scales[8];
    for (int64_t i = 0; i < n / QK_K; ++i) {
        const float* xb = x + i * QK_K;
        float sum_x2 = 0.0f;
        for (int l = 0; l < QK_K; ++l) sum_x2 = fmaf(xb[l], xb[l], sum_x2);
        float sigma2 = 2.0f * sum_x2 / (float)QK_K;
        for (int j = 0; j < 8; ++j) {
            const float* sub = xb + 32 * j;
            const float* qw = quant_weights + QK_K * i + 32 * j;
            for (int l = 0; l < 32; ++l) weights[l] = qw[l] * std::sqrt(sigma2 + sub[l] * sub[l]);
            float sumw = 0.0f;
            for (int l = 0; l < 32; ++l) sumw += weights[l];
            sw[j] = sumw;
            scales[j] = make_qkx_quants(true, 32, nmax, sub, weights, L + 32 * j, &mins[j], Laux,
                                        -0.9f, 0.05f, 36, false);
        }
        float d_block = make_qp_quants(8, 63, scales, Ls, sw);
        float m_block = make_qp_quants(8, 63, mins, Lm, sw);
        uint8_t sp[K_SCALE_SIZE] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t ls = Ls[j], lm = Lm[j];
            if (is_q5) { if (ls > 63) ls = 63; if (lm > 63) lm = 63; }   // q5_k.rs:301-302
            pack_scale_min_k4(j, sp, ls, lm);
        }
        uint16_t d_h = f32_to_f16(d_block), dmin_h = f32_to_f16(m_block);
        k45_reencode(xb, d_h, dmin_h, sp, L, nmax);
        if (is_q5) q5_k_emit(d_h, dmin_h, sp, L, out + i * bb);
        else       q4_k_emit(d_h, dmin_h, sp, L, out + i * bb);
    }
}

// ---- Q6_K ------------------------------------------------------------------------------------
// q6_k.rs:40-151; qw == nullptr is the reference's empty slice.
void q6_k_block(const float* xb, const float* qw, uint8_t* o) {
    int8_t L[QK_K]; float scales[16];
    std::memset(L, 0, sizeof L);
    float max_scale = 0.0f, max_abs_scale = 0.0f;
    for (int ib = 0; ib < 16; ++ib) {
        float scale = make_qx_quants(16, 32, xb + 16 * ib, L + 16 * ib, 1, qw ? qw + 16 * ib : nullptr);
        scales[ib] = scale;
        float a = std::fabs(scale);
        if (a > max_abs_scale) { max_abs_scale = a; max_scale = scale; }
    }
    std::memset(o, 0, 210);
    if (max_abs_scale < GROUP_MAX_EPS) return;
    float iscale = -128.0f / max_scale;
    uint16_t d_h = f32_to_f16(1.0f / iscale);
    int8_t sc[16];
    for (int ib = 0; ib < 16; ++ib) sc[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
    float d_back = f16_to_f32(d_h);
    for (int j = 0; j < 16; ++j) {
        float d = d_back * (float)sc[j];
        if (d == 0.0f) continue;
        for (int ii = 0; ii < 16; ++ii) {
            int l = clampi(nearest_int(xb[16 * j + ii] / d), -32, 31);
            L[16 * j + ii] = (int8_t)(l + 32);
        }
    }
    uint8_t* ql = o; uint8_t* qh = o + 128;
    for (int j = 0; j < QK_K; j += 128) {
        for (int l = 0; l < 32; ++l) {
            uint8_t a = (uint8_t)L[j + l], b = (uint8_t)L[j + l + 32];
            uint8_t c = (uint8_t)L[j + l + 64], d = (uint8_t)L[j + l + 96];
            ql[l] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
            ql[l + 32] = (uint8_t)((b & 0xF) | ((d & 0xF) << 4));
            qh[l] = (uint8_t)((a >> 4) | ((b >> 4) << 2) | ((c >> 4) << 4) | ((d >> 4) << 6));
        }
        ql += 64; qh += 32;
    }
    for (int ib = 0; ib < 16; ++ib) o[192 + ib] = (uint8_t)sc[ib];
    put_f16(o + 208, d_h);
}

// ---- geometry (ggml_type.rs:60-133) ----------------------------------------------------------
enum : uint32_t { T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ4_NL = 20 };

bool geometry(uint32_t t, int* block_elems, int* block_bytes) {
    switch (t) {
        case T_Q4_0: *block_elems = 32; *block_bytes = 18; return true;
        case T_Q8_0: *block_elems = 32; *block_bytes = 34; return true;
        case T_Q4_K: *block_elems = 256; *block_bytes = 144; return true;
        case T_Q5_K: *block_elems = 256; *block_bytes = 176; return true;
        case T_Q6_K: *block_elems = 256; *block_bytes = 210; return true;
        case T_Q4_1: *block_elems = 32; *block_bytes = 20; return true;     // ggml_type.rs:100-105
        case T_Q5_0: *block_elems = 32; *block_bytes = 22; return true;
        case T_Q5_1: *block_elems = 32; *block_bytes = 24; return true;
        case T_IQ4_NL: *block_elems = 32; *block_bytes = 18; return true;
        default: return false;
    }
}

// ---- dequantise one block (inverse of the re-encode step; see header) -------------------------
void dequant_block(uint32_t t, const uint8_t* b, float* y) {
    switch (t) {
    case T_Q4_0: {   // q4_0.rs:47-64
        float d = f16_to_f32(get_u16(b));
        for (int j = 0; j < 16; ++j) {
            y[j] = (float)((int)(b[2 + j] & 15) - 8) * d;
            y[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d;
        }
    } break;
    case T_Q8_0: {   // q8_0.rs:59-67
        float d = f16_to_f32(get_u16(b));
        for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)b[2 + j] * d;
    } break;
    case T_Q4_K: {   // q4_k.rs:183-215
        float d = f16_to_f32(get_u16(b)), dmin = f16_to_f32(get_u16(b + 2));
        const uint8_t* sc = b + 4; const uint8_t* qs = b + 16;
        for (int c = 0; c < 4; ++c) {
            uint8_t s1, m1, s2, m2;
            get_scale_min_k4(2 * c, sc, &s1, &m1);
            get_scale_min_k4(2 * c + 1, sc, &s2, &m2);
            float d1 = d * (float)s1, mm1 = dmin * (float)m1;
            float d2 = d * (float)s2, mm2 = dmin * (float)m2;
            for (int l = 0; l < 32; ++l) {
                y[64 * c + l] = d1 * (float)(qs[32 * c + l] & 15) - mm1;
                y[64 * c + 32 + l] = d2 * (float)(qs[32 * c + l] >> 4) - mm2;
            }
        }
    } break;
    case T_Q5_K: {   // q5_k.rs:100-158
        float d = f16_to_f32(get_u16(b)), dmin = f16_to_f32(get_u16(b + 2));
        const uint8_t* sc = b + 4; const uint8_t* qh = b + 16; const uint8_t* qs = b + 48;
        for (int c = 0; c < 4; ++c) {
            uint8_t s1, m1, s2, m2;
            get_scale_min_k4(2 * c, sc, &s1, &m1);
            get_scale_min_k4(2 * c + 1, sc, &s2, &m2);
            float d1 = d * (float)s1, mm1 = dmin * (float)m1;
            float d2 = d * (float)s2, mm2 = dmin * (float)m2;
            for (int l = 0; l < 32; ++l) {
                int q1 = (qs[32 * c + l] & 15) + 16 * ((qh[l] >> (2 * c)) & 1);
                int q2 = (qs[32 * c + l] >> 4) + 16 * ((qh[l] >> (2 * c + 1)) & 1);
                y[64 * c + l] = d1 * (float)q1 - mm1;
                y[64 * c + 32 + l] = d2 * (float)q2 - mm2;
            }
        }
    } break;
    case T_Q6_K: {   // q6_k.rs:96-143
        const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192);
        float d = f16_to_f32(get_u16(b + 208));
        for (int n = 0; n < 2; ++n)
            for (int l = 0; l < 32; ++l)
                for (int k = 0; k < 4; ++k) {
                    int lo = k < 2 ? (ql[64 * n + l + 32 * k] & 15) : (ql[64 * n + l + 32 * (k - 2)] >> 4);
                    int hi = (qh[32 * n + l] >> (2 * k)) & 3;
                    int q = (lo | (hi << 4)) - 32;
                    int e = 128 * n + 32 * k + l;
                    y[e] = (d * (float)sc[e / 16]) * (float)q;
                }
    } break;
    // The 32-element fallback formats: the value each code stands for is the one the quantizers'
    // own error terms use -- scale*L + min in make_qkx3_quants (common.rs:339-343, Q4_1 / Q5_1), the
    // symmetric grid of make_qx_quants shifted by nmax (Q5_0, q5_0.rs:80-100) and d * values[L] for
    // IQ4_NL (iq4_nl.rs first pass).  d*q is exact in f32, so fused or not the one addition rounds alike.
    case T_Q4_1: {
        float d = f16_to_f32(get_u16(b)), m = f16_to_f32(get_u16(b + 2));
        for (int j = 0; j < 16; ++j) {
            y[j] = d * (float)(b[4 + j] & 15) + m;
            y[j + 16] = d * (float)(b[4 + j] >> 4) + m;
        }
    } break;
    case T_Q5_0: {
        float d = f16_to_f32(get_u16(b));
        uint32_t qh = get_u32(b + 2);
        for (int j = 0; j < 16; ++j) {
            int q0 = (b[6 + j] & 15) | (int)(((qh >> j) & 1u) << 4);
            int q1 = (b[6 + j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
            y[j] = (float)(q0 - 16) * d;
            y[j + 16] = (float)(q1 - 16) * d;
        }
    } break;
    case T_Q5_1: {
        float d = f16_to_f32(get_u16(b)), m = f16_to_f32(get_u16(b + 2));
        uint32_t qh = get_u32(b + 4);
        for (int j = 0; j < 16; ++j) {
            int q0 = (b[8 + j] & 15) | (int)(((qh >> j) & 1u) << 4);
            int q1 = (b[8 + j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
            y[j] = d * (float)q0 + m;
            y[j + 16] = d * (float)q1 + m;
        }
    } break;
    case T_IQ4_NL: {
        float d = f16_to_f32(get_u16(b));
        for (int j = 0; j < 16; ++j) {
            y[j] = d * (float)KVALUES_IQ4NL[b[2 + j] & 15];
            y[j + 16] = d * (float)KVALUES_IQ4NL[b[2 + j] >> 4];
        }
    } break;
    default: break;
    }
}

}  // namespace

extern "C" {

int oracle_block_geometry(uint32_t ggml_type, int* block_elems, int* block_bytes) {
    return geometry(ggml_type, block_elems, block_bytes) ? 0 : -1;
}

// ggml_type.rs:131-133
int64_t oracle_row_bytes(uint32_t ggml_type, int64_t k) {
    int be, bb;
    if (!geometry(ggml_type, &be, &bb) || k % be) return -1;
    return k / be * bb;
}

void oracle_f16_round_trip(const float* in, float* out, int64_t n) {   // orchestrator.rs:536-550
    for (int64_t i = 0; i < n; ++i) out[i] = f16_to_f32(f32_to_f16(in[i]));
}
uint16_t oracle_f32_to_f16(float f) { return f32_to_f16(f); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
int oracle_nearest_int(float f) { return nearest_int(f); }

// Quantize n_rows x n_per_row f32 -> blocks.  imatrix is null or n_per_row long (reused per row).
// `threads` > 1 splits rows over OpenMP threads; every row is independent in all five formats
// (Q4_0's and Q8_0's whole-buffer loops are block-local), so the bytes do not depend on it.
int oracle_quantize(uint32_t ggml_type, const float* src, int64_t n_rows, int64_t n_per_row,
                    const float* imatrix, uint8_t* out, int threads) {
    int be, bb;
    if (!geometry(ggml_type, &be, &bb) || n_per_row % be) return -1;
    const int64_t rb = n_per_row / be * bb;
    (void)threads;
#pragma omp parallel for schedule(dynamic, 4) num_threads(threads > 0 ? threads : 1)
    for (int64_t r = 0; r < n_rows; ++r) {
        const float* x = src + r * n_per_row;
        uint8_t* o = out + r * rb;
        switch (ggml_type) {
        case T_Q4_0: imatrix ? q4_0_row_impl(x, imatrix, n_per_row, o) : q4_0_row_ref(x, n_per_row, o); break;
        case T_Q8_0: q8_0_blocks(x, n_per_row, o); break;
        case T_Q4_K: imatrix ? k45_row_impl(x, imatrix, n_per_row, o, false) : k45_row_ref(x, n_per_row, o, false); break;
        case T_Q5_K: imatrix ? k45_row_impl(x, imatrix, n_per_row, o, true) : k45_row_ref(x, n_per_row, o, true); break;
        case T_Q6_K:
            for (int64_t i = 0; i < n_per_row / QK_K; ++i)
                q6_k_block(x + i * QK_K, imatrix ? imatrix + i * QK_K : nullptr, o + i * 210);
            break;
        case T_Q4_1: q4_1_row(x, imatrix, n_per_row, o); break;
        case T_Q5_0: q5_0_row(x, imatrix, n_per_row, o); break;
        case T_Q5_1: q5_1_row(x, imatrix, n_per_row, o); break;
        case T_IQ4_NL:
            for (int64_t i = 0; i < n_per_row / 32; ++i)
                iq4_nl_block(x + 32 * i, imatrix ? imatrix + 32 * i : nullptr, o + 18 * i);
            break;
        }
    }
    return 0;
}

// gpu_full_attn.rs:427-451: d = amax/7 (1.0 for a zero block), q = clamp(round(x/d), -8, 7) + 8.
int oracle_encode_q4_0_simple(const float* vals, int64_t n, uint8_t* out) {
    if (n % 32) return -1;
    for (int64_t b = 0; b < n / 32; ++b) {
        const float* blk = vals + b * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(blk[j]));   // f32::max
        float d = amax > 0.0f ? amax / 7.0f : 1.0f;
        uint8_t* o = out + b * 18;
        put_f16(o, f32_to_f16(d));
        for (int j = 0; j < 16; ++j) {
            auto q = [&](float v) -> uint8_t {
                float r = std::round(v / d);
                r = r < -8.0f ? -8.0f : (r > 7.0f ? 7.0f : r);      // NaN passes through clamp
                return (uint8_t)(sat_i8(r) + 8);
            };
            o[2 + j] = (uint8_t)((q(blk[j]) & 0x0F) | ((q(blk[j + 16]) & 0x0F) << 4));
        }
    }
    return 0;
}

int oracle_dequantize(uint32_t ggml_type, const uint8_t* blocks, int64_t n_elems, float* out,
                      int threads) {
    int be, bb;
    if (!geometry(ggml_type, &be, &bb) || n_elems % be) return -1;
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (int64_t i = 0; i < n_elems / be; ++i) dequant_block(ggml_type, blocks + i * bb, out + i * be);
    return 0;
}

// ffn.rs:38-50: out[i,j] = sum_k lhs[i,k]*rhs[j,k], sequential k, f32, unfused.
void oracle_matmul_a_by_bt(const float* lhs, const float* rhs, int64_t m, int64_t k, int64_t n,
                           float* out, int threads) {
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (int64_t j = 0; j < n; ++j)
        for (int64_t i = 0; i < m; ++i) {
            float acc = 0.0f;
            const float* a = lhs + i * k; const float* b = rhs + j * k;
            for (int64_t kk = 0; kk < k; ++kk) acc += a[kk] * b[kk];
            out[i * n + j] = acc;
        }
}

// The accuracy yardstick: the same contraction in f64 on f32 operands.
void oracle_matmul_f64(const float* lhs, const float* rhs, int64_t m, int64_t k, int64_t n,
                       double* out, int threads) {
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (int64_t j = 0; j < n; ++j)
        for (int64_t i = 0; i < m; ++i) {
            double acc = 0.0;
            const float* a = lhs + i * k; const float* b = rhs + j * k;
            for (int64_t kk = 0; kk < k; ++kk) acc += (double)a[kk] * (double)b[kk];
            out[i * n + j] = acc;
        }
}

// The reference's CPU path for one quantized matmul: dequantise W to f32, then matmul_a_by_bt.
// `w_f32` is caller scratch of n*k floats.  Returns seconds spent in (dequant, matmul) through
// t_out[0], t_out[1] when t_out is non-null.
int oracle_qmatmul(uint32_t ggml_type, const uint8_t* w, const float* x, int64_t m, int64_t n,
                   int64_t k, float* w_f32, float* y, int threads, double* t_out) {
    double t0 = 0, t1 = 0, t2 = 0;
#ifdef _OPENMP
    t0 = omp_get_wtime();
#endif
    if (oracle_dequantize(ggml_type, w, n * k, w_f32, threads)) return -1;
#ifdef _OPENMP
    t1 = omp_get_wtime();
#endif
    oracle_matmul_a_by_bt(x, w_f32, m, k, n, y, threads);
#ifdef _OPENMP
    t2 = omp_get_wtime();
#endif
    if (t_out) { t_out[0] = t1 - t0; t_out[1] = t2 - t1; }
    return 0;
}

// Expert-routed product, the semantics of quantized_matmul_id_ggml as its callers use it
// (gpu_ffn.rs:2606-2618, forward_mlx.rs:5285-5292): out[t*top_k+s, :] =
// x[t, :] . dequant(W[ids[t*top_k+s]])^T, expert slice at byte offset id*expert_stride.
int oracle_qmatmul_id(uint32_t ggml_type, const uint8_t* w_stacked, uint64_t expert_stride,
                      const float* x, const uint32_t* ids, int64_t n_tokens, int64_t top_k,
                      int64_t n, int64_t k, int64_t n_experts, float* y, int threads) {
    int be, bb;
    if (!geometry(ggml_type, &be, &bb) || k % be) return -1;
    const int64_t rb = k / be * bb;
    for (int64_t r = 0; r < n_tokens * top_k; ++r) if (ids[r] >= (uint64_t)n_experts) return -2;
    (void)threads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        std::vector<float> row((size_t)k);
#pragma omp for schedule(dynamic, 8) collapse(2)
        for (int64_t r = 0; r < n_tokens * top_k; ++r)
            for (int64_t j = 0; j < n; ++j) {
                const uint8_t* wr = w_stacked + (uint64_t)ids[r] * expert_stride + j * rb;
                for (int64_t b = 0; b < k / be; ++b) dequant_block(ggml_type, wr + b * bb, row.data() + b * be);
                const float* a = x + (r / top_k) * k;
                float acc = 0.0f;
                for (int64_t kk = 0; kk < k; ++kk) acc += a[kk] * row[kk];
                y[r * n + j] = acc;
            }
    }
    return 0;
}

// gpu_ffn.rs:1879-1924.  Stable descending sort on probability: ties keep the lower index first.
void oracle_softmax_topk_renorm(const float* logits, int64_t seq_len, int64_t num_experts,
                                int64_t topk, uint32_t* out_idx, float* out_w) {
    std::vector<float> ev((size_t)num_experts);
    std::vector<int64_t> order((size_t)num_experts);
    for (int64_t t = 0; t < seq_len; ++t) {
        const float* row = logits + t * num_experts;
        float max_v = -INFINITY;
        for (int64_t e = 0; e < num_experts; ++e) max_v = std::fmax(max_v, row[e]);
        float denom = 0.0f;
        for (int64_t e = 0; e < num_experts; ++e) { ev[e] = std::exp(row[e] - max_v); }
        for (int64_t e = 0; e < num_experts; ++e) denom += ev[e];
        float inv_d = denom > 1e-20f ? 1.0f / denom : 1.0f;
        for (int64_t e = 0; e < num_experts; ++e) ev[e] *= inv_d;
        std::iota(order.begin(), order.end(), 0);
        // The reference sorts stably with partial_cmp().unwrap_or(Equal) (gpu_ffn.rs:1903-1908), which is
        // not a total order once a NaN is present.  The order is made total here the way the CUDA kernel
        // does it: a NaN ranks below every number, equal keys keep the lower index first.
        auto key = [&](int64_t i) { return ev[i] != ev[i] ? -1.0f : ev[i]; };
        std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return key(b) < key(a); });
        float sum_sel = 0.0f;
        for (int64_t s = 0; s < topk; ++s) sum_sel += ev[order[s]];
        float inv_sum = sum_sel > 1e-20f ? 1.0f / sum_sel : 1.0f / (float)topk;
        for (int64_t s = 0; s < topk; ++s) {
            out_idx[t * topk + s] = (uint32_t)order[s];
            out_w[t * topk + s] = ev[order[s]] * inv_sum;
        }
    }
}

// ffn.rs:24-30
static inline float silu_ref(float x) { return x / (1.0f + std::exp(-x)); }
static inline float sigmoid_ref(float x) { return 1.0f / (1.0f + std::exp(-x)); }

// dense_swiglu_cpu_ref (ffn.rs:91-112): y = down @ (silu(gate @ x) * (up @ x)); all f32, weights
// [out, in] row-major (already dequantised), x [seq, h], y [seq, h].
void oracle_dense_swiglu(const float* x, const float* gate, const float* up, const float* down, int64_t seq,
                         int64_t h, int64_t m, float* y, int threads) {
    std::vector<float> a((size_t)seq * m), b((size_t)seq * m);
    oracle_matmul_a_by_bt(x, gate, seq, h, m, a.data(), threads);
    oracle_matmul_a_by_bt(x, up, seq, h, m, b.data(), threads);
    for (int64_t i = 0; i < seq * m; ++i) a[i] = silu_ref(a[i]) * b[i];
    oracle_matmul_a_by_bt(a.data(), down, seq, m, h, y, threads);
}

// moe_ffn_cpu_ref (ffn.rs:179-336).  Router logits, softmax, stable top-k, renormalise, per-expert
// SwiGLU, weighted sum; plus the sigmoid-gated shared expert when m_sh > 0.
void oracle_moe_ffn(const float* x, const float* router, const float* eg, const float* eu, const float* ed,
                    const float* sh_logit, const float* sg, const float* su, const float* sd, int64_t seq, int64_t h,
                    int64_t ne, int64_t topk, int64_t m_moe, int64_t m_sh, float* out) {
    std::vector<float> logits((size_t)ne), ex((size_t)ne), probs((size_t)ne), a((size_t)m_moe), b((size_t)m_moe),
        yv((size_t)h), moe((size_t)h), as((size_t)(m_sh > 0 ? m_sh : 1)), bs((size_t)(m_sh > 0 ? m_sh : 1));
    std::vector<int64_t> order((size_t)ne);
    for (int64_t t = 0; t < seq; ++t) {
        const float* xt = x + t * h;
        for (int64_t e = 0; e < ne; ++e) {
            float acc = 0.0f;
            for (int64_t i = 0; i < h; ++i) acc += router[e * h + i] * xt[i];
            logits[e] = acc;
        }
        float mx = -INFINITY;
        for (int64_t e = 0; e < ne; ++e) mx = std::fmax(mx, logits[e]);
        float denom = 0.0f;
        for (int64_t e = 0; e < ne; ++e) { ex[e] = std::exp(logits[e] - mx); denom += ex[e]; }
        for (int64_t e = 0; e < ne; ++e) probs[e] = ex[e] / denom;
        std::iota(order.begin(), order.end(), 0);
        std::stable_sort(order.begin(), order.end(), [&](int64_t p, int64_t q) { return probs[q] < probs[p]; });
        float rs = 0.0f;
        for (int64_t s = 0; s < topk; ++s) rs += probs[order[s]];
        std::fill(moe.begin(), moe.end(), 0.0f);
        for (int64_t s = 0; s < topk; ++s) {
            const int64_t e = order[s];
            const float w = rs > 1e-20f ? probs[e] / rs : 1.0f / (float)topk;
            const float* g = eg + e * m_moe * h; const float* u = eu + e * m_moe * h; const float* d = ed + e * h * m_moe;
            for (int64_t i = 0; i < m_moe; ++i) {
                float ga = 0.0f, ua = 0.0f;
                for (int64_t j = 0; j < h; ++j) ga += g[i * h + j] * xt[j];
                for (int64_t j = 0; j < h; ++j) ua += u[i * h + j] * xt[j];
                a[i] = silu_ref(ga) * ua;
            }
            for (int64_t i = 0; i < h; ++i) {
                float acc = 0.0f;
                for (int64_t j = 0; j < m_moe; ++j) acc += d[i * m_moe + j] * a[j];
                moe[i] += w * acc;
            }
        }
        if (m_sh > 0) {
            float lg = 0.0f;
            for (int64_t i = 0; i < h; ++i) lg += sh_logit[i] * xt[i];
            const float gv = sigmoid_ref(lg);
            for (int64_t i = 0; i < m_sh; ++i) {
                float ga = 0.0f, ua = 0.0f;
                for (int64_t j = 0; j < h; ++j) ga += sg[i * h + j] * xt[j];
                for (int64_t j = 0; j < h; ++j) ua += su[i * h + j] * xt[j];
                as[i] = silu_ref(ga) * ua;
            }
            for (int64_t i = 0; i < h; ++i) {
                float acc = 0.0f;
                for (int64_t j = 0; j < m_sh; ++j) acc += sd[i * m_sh + j] * as[j];
                out[t * h + i] = moe[i] + gv * acc;
            }
        } else {
            for (int64_t i = 0; i < h; ++i) out[t * h + i] = moe[i];
        }
    }
    (void)b; (void)bs; (void)yv;
}

// mulberry32 streams of the fixture generator (scripts/ggml_quants_harness/gen.c:24-50).
static inline uint32_t mulberry32_step(uint32_t* state) {
    *state += 0x6D2B79F5u;
    uint32_t t = *state;
    t = (t ^ (t >> 15)) * (t | 1u);
    t ^= t + (t ^ (t >> 7)) * (t | 61u);
    return t ^ (t >> 14);
}
void oracle_mulberry32_uniform(float* out, int64_t n, uint32_t seed) {
    uint32_t s = seed;
    for (int64_t i = 0; i < n; ++i) out[i] = ((float)mulberry32_step(&s) / (float)0xFFFFFFFFu) * 2.0f - 1.0f;
}
void oracle_mulberry32_imatrix(float* out, int64_t n, uint32_t seed) {
    uint32_t s = seed;
    for (int64_t i = 0; i < n; ++i) {
        float v = ((float)mulberry32_step(&s) / (float)0xFFFFFFFFu) * 2.0f - 1.0f;
        out[i] = std::fabs(v) + 1e-3f;
    }
}

// Overrides an inherited OMP_NUM_THREADS (launchers such as torchrun export OMP_NUM_THREADS=1).
void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
