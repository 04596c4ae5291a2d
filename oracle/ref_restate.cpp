// TEST INFRASTRUCTURE — CPU restatement of the pieces of cretz/thinfer's quantised-linear
// path that the reference itself pins with unit tests. Not a product path.
//
// The NVFP4 oracle (nvfp4_oracle.cpp) borrows its conventions from these routines; they
// are restated here so that the borrowing can be checked against the reference's own
// known-answer tests (see tests/test_oracle_pins.py). Each function cites the reference
// lines it follows. f16 narrowing follows the `half` crate 2.7.1 behaviour (IEEE RNE with
// subnormals) that thinfer-core/src/weight.rs:269-336 and
// thinfer-core/src/ops/weight_prep.rs:52-80 pin.

#include <cmath>
#include <cstdint>
#include <cstring>

namespace {
inline uint32_t f32_bits(float x) { uint32_t b; std::memcpy(&b, &x, 4); return b; }
inline float bits_f32(uint32_t b) { float x; std::memcpy(&x, &b, 4); return x; }

// IEEE binary16 <- binary32, round-to-nearest-even, subnormals kept.
inline uint16_t f16_from_f32(float x) {
    uint32_t b = f32_bits(x);
    uint32_t sign = (b >> 16) & 0x8000u;
    uint32_t abs = b & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return uint16_t(sign | 0x7E00u | ((abs >> 13) & 0x3FFu));  // NaN
    if (abs >= 0x47800000u) return uint16_t(sign | 0x7C00u);                          // >= 65536 -> inf
    if (abs < 0x33000000u) return uint16_t(sign);                                     // < 2^-25 -> 0
    int e = int(abs >> 23) - 127;
    uint32_t mant = (abs & 0x7FFFFFu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t q = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    uint32_t out = (e < -14) ? q : ((uint32_t(e + 15) << 10) + (q - 0x400u));
    return uint16_t(sign | out);  // mantissa carry propagates into the exponent, inf at 0x7C00
}
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = uint32_t(h & 0x8000u) << 16;
    int e = (h >> 10) & 0x1F;
    uint32_t m = h & 0x3FFu;
    if (e == 0) return bits_f32(sign) + (sign ? -1.0f : 1.0f) * std::ldexp(float(m), -24);
    if (e == 31) return bits_f32(sign | 0x7F800000u | (m << 13));
    return bits_f32(sign | (uint32_t(e + 112) << 23) | (m << 13));
}
// Rust f32::round: half away from zero.
inline float round_half_away(float v) { return std::round(v); }
}  // namespace

extern "C" {

uint16_t ref_f16_from_f32(float x) { return f16_from_f32(x); }
float ref_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// LCG of the reference's conformance tests (thinfer-conformance/tests/q4_0_matmul.rs:56-61):
// s = s*6364136223846793005 + 1 ; r = (s>>33) as u32 as f32 / u32::MAX as f32 ; r*2-1.
void ref_lcg_fill(float* out, int64_t n, uint64_t* state, float amp) {
    uint64_t s = *state;
    for (int64_t i = 0; i < n; ++i) {
        s = s * 6364136223846793005ull + 1ull;
        float r = float(uint32_t(s >> 33)) / float(0xFFFFFFFFu);
        out[i] = (r * 2.0f - 1.0f) * amp;
    }
    *state = s;
}

// thinfer-core/src/quant.rs:735-755 (quantize_row_q8_0): 34-byte blocks, f16 d + 32 i8.
void ref_quantize_row_q8_0(const float* src, int64_t n, uint8_t* dst) {
    for (int64_t b = 0; b < n / 32; ++b) {
        const float* x = src + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(x[i]));
        float scale = amax / 127.0f;
        float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
        uint16_t h = f16_from_f32(scale);
        dst[b * 34] = uint8_t(h & 0xFF);
        dst[b * 34 + 1] = uint8_t(h >> 8);
        for (int i = 0; i < 32; ++i) {
            float q = round_half_away(x[i] * inv);
            q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
            dst[b * 34 + 2 + i] = uint8_t(int8_t(q));
        }
    }
}

// thinfer-core/src/quant.rs:169-194 (encode_q8_0_from_bf16): source is bf16 bits.
void ref_encode_q8_0_from_bf16(const uint16_t* src, int64_t n, uint8_t* dst) {
    for (int64_t b = 0; b < n / 32; ++b) {
        float x[32];
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) {
            x[i] = bits_f32(uint32_t(src[b * 32 + i]) << 16);
            amax = std::fmax(amax, std::fabs(x[i]));
        }
        float d = amax / 127.0f;
        float id = d == 0.0f ? 0.0f : 1.0f / d;
        uint16_t h = f16_from_f32(d);
        dst[b * 34] = uint8_t(h & 0xFF);
        dst[b * 34 + 1] = uint8_t(h >> 8);
        for (int i = 0; i < 32; ++i) dst[b * 34 + 2 + i] = uint8_t(int8_t(round_half_away(x[i] * id)));
    }
}

// thinfer-core/src/quant.rs:709-733 (dequantize_row_q8_0).
void ref_dequantize_row_q8_0(const uint8_t* src, int64_t n, float* dst) {
    for (int64_t b = 0; b < n / 32; ++b) {
        float scale = f16_to_f32(uint16_t(src[b * 34] | (src[b * 34 + 1] << 8)));
        for (int i = 0; i < 32; ++i) dst[b * 32 + i] = float(int8_t(src[b * 34 + 2 + i])) * scale;
    }
}

// thinfer-core/src/quant.rs:784-811 (quantize_row_q4_0): 18-byte blocks; byte j packs
// element j (low nibble) and j+16 (high nibble).
void ref_quantize_row_q4_0(const float* src, int64_t n, uint8_t* dst) {
    for (int64_t b = 0; b < n / 32; ++b) {
        const float* x = src + b * 32;
        float amax = 0.0f, smax = 0.0f;
        for (int i = 0; i < 32; ++i)
            if (std::fabs(x[i]) > amax) { amax = std::fabs(x[i]); smax = x[i]; }
        float d = smax / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint16_t h = f16_from_f32(d);
        dst[b * 18] = uint8_t(h & 0xFF);
        dst[b * 18 + 1] = uint8_t(h >> 8);
        for (int j = 0; j < 16; ++j) {
            int a0 = int(std::floor(x[j] * id + 8.5f)), a1 = int(std::floor(x[j + 16] * id + 8.5f));
            a0 = a0 < 0 ? 0 : (a0 > 15 ? 15 : a0);
            a1 = a1 < 0 ? 0 : (a1 > 15 ? 15 : a1);
            dst[b * 18 + 2 + j] = uint8_t(a0 | (a1 << 4));
        }
    }
}

// thinfer-core/src/quant.rs:757-782 (dequantize_row_q4_0).
void ref_dequantize_row_q4_0(const uint8_t* src, int64_t n, float* dst) {
    for (int64_t b = 0; b < n / 32; ++b) {
        float scale = f16_to_f32(uint16_t(src[b * 18] | (src[b * 18 + 1] << 8)));
        for (int j = 0; j < 16; ++j) {
            uint8_t by = src[b * 18 + 2 + j];
            dst[b * 32 + j] = float(int(by & 0xF) - 8) * scale;
            dst[b * 32 + j + 16] = float(int(by >> 4) - 8) * scale;
        }
    }
}

// thinfer-core/src/ops/act_quant.rs:121-151 and
// thinfer-conformance/tests/i8_common/mod.rs:245-272 (quant_block_to_i8): asymmetric
// int8 per 32-block; the parameters are narrowed to f16 BEFORE the codes are computed.
void ref_act_quant_i8(const float* a, int64_t rows, int64_t k, int8_t* q, float* params /*[rows*k/32*2]*/) {
    int64_t nb = k / 32;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            const float* x = a + r * k + b * 32;
            float mn = INFINITY, mx = -INFINITY;
            for (int i = 0; i < 32; ++i) { if (x[i] < mn) mn = x[i]; if (x[i] > mx) mx = x[i]; }
            float range = mx - mn;
            float s_raw = range <= 0.0f ? 1.0e-30f : range / 254.0f;
            float z_raw = mn + 127.0f * s_raw;
            float s = f16_to_f32(f16_from_f32(s_raw)), z = f16_to_f32(f16_from_f32(z_raw));
            float inv = 1.0f / s;
            for (int i = 0; i < 32; ++i) {
                float v = round_half_away((x[i] - z) * inv);
                v = v < -127.0f ? -127.0f : (v > 127.0f ? 127.0f : v);
                q[r * k + b * 32 + i] = int8_t(int(v));
            }
            params[2 * (r * nb + b)] = s;
            params[2 * (r * nb + b) + 1] = z;
        }
}

// thinfer-conformance/tests/matmul_i8.rs:76-116 (cpu_matmul_i8_ref).
void ref_matmul_i8(const int8_t* a, const float* a_scale, const float* a_zero, const int8_t* b,
                   const float* b_scale, int64_t m, int64_t n, int64_t k, float* out) {
    int64_t nb = k / 32;
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (int64_t t = 0; t < nb; ++t) {
                int32_t dot = 0, qsum = 0;
                for (int kk = 0; kk < 32; ++kk) {
                    int32_t av = a[i * k + t * 32 + kk], bv = b[j * k + t * 32 + kk];
                    dot += av * bv;
                    qsum += bv;
                }
                float sa = a_scale[i * nb + t], za = a_zero[i * nb + t], sb = b_scale[j * nb + t];
                acc += float(dot) * sa * sb + za * sb * float(qsum);
            }
            out[i * n + j] = acc < -65504.0f ? -65504.0f : (acc > 65504.0f ? 65504.0f : acc);
        }
}

// thinfer-core/src/ops/layernorm.rs:58-82 (f32 activations) and :95-125 (packed bf16): no affine,
// one row at a time, both sums SEQUENTIAL in f32 (mean first, then the squared deviations), then
// (x - mean) * inverseSqrt(sum_sq / dim + eps). bf16 = 1 reads bf16 bits and rounds the result to
// bf16 (RNE) like the packed kernel's pack_bf16x2; bf16 = 0 is the f32 kernel.
static inline float rs_bf16_f32(uint16_t h) { uint32_t u = uint32_t(h) << 16; float f; std::memcpy(&f, &u, 4); return f; }
static inline uint16_t rs_bf16_rne(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((u >> 16) | 0x40);
    return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
void ref_layernorm(const void* x, int bf16, int64_t rows, int64_t dim, float eps, void* out) {
    const float* xf = static_cast<const float*>(x);
    const uint16_t* xh = static_cast<const uint16_t*>(x);
    for (int64_t r = 0; r < rows; ++r) {
        float sum = 0.0f;
        for (int64_t i = 0; i < dim; ++i) sum = sum + (bf16 ? rs_bf16_f32(xh[r * dim + i]) : xf[r * dim + i]);
        float mean = sum / float(dim);
        float sum_sq = 0.0f;
        for (int64_t i = 0; i < dim; ++i) {
            float d = (bf16 ? rs_bf16_f32(xh[r * dim + i]) : xf[r * dim + i]) - mean;
            sum_sq = sum_sq + d * d;
        }
        float inv = 1.0f / std::sqrt(sum_sq / float(dim) + eps);
        for (int64_t i = 0; i < dim; ++i) {
            float v = ((bf16 ? rs_bf16_f32(xh[r * dim + i]) : xf[r * dim + i]) - mean) * inv;
            if (bf16) static_cast<uint16_t*>(out)[r * dim + i] = rs_bf16_rne(v);
            else static_cast<float*>(out)[r * dim + i] = v;
        }
    }
}

// thinfer-core/src/ops/bcast_modulate.rs:1-3,93-102: out[i] = x[i] * (s[i % C] + bias) + t[i % C];
// AdaLN modulation norm(x) * (1 + scale) + shift with bias = 1.
void ref_bcast_modulate(const void* x, const void* s, const void* t, int bf16, int64_t n, int64_t c, float bias, void* out) {
    for (int64_t i = 0; i < n; ++i) {
        float xv, sv, tv;
        if (bf16) {
            xv = rs_bf16_f32(static_cast<const uint16_t*>(x)[i]);
            sv = rs_bf16_f32(static_cast<const uint16_t*>(s)[i % c]);
            tv = rs_bf16_f32(static_cast<const uint16_t*>(t)[i % c]);
        } else {
            xv = static_cast<const float*>(x)[i];
            sv = static_cast<const float*>(s)[i % c];
            tv = static_cast<const float*>(t)[i % c];
        }
        float v = xv * (sv + bias) + tv;
        if (bf16) static_cast<uint16_t*>(out)[i] = rs_bf16_rne(v);
        else static_cast<float*>(out)[i] = v;
    }
}

// The fused form of the two dispatches above (what the device kernel computes): LayerNorm then
// modulate on one row, bf16 in, bf16 out. chain = 1 rounds the LayerNorm result to bf16 before the
// modulation, as the reference's two dispatches do; chain = 0 keeps it in f32. s == null skips the
// modulation (out = bf16(LayerNorm(x))).
void ref_norm_modulate_bf16(const uint16_t* x, const uint16_t* s, const uint16_t* t, int64_t rows, int64_t dim, float eps,
                            float bias, int chain, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float sum = 0.0f;
        for (int64_t i = 0; i < dim; ++i) sum = sum + rs_bf16_f32(x[r * dim + i]);
        float mean = sum / float(dim);
        float sum_sq = 0.0f;
        for (int64_t i = 0; i < dim; ++i) {
            float d = rs_bf16_f32(x[r * dim + i]) - mean;
            sum_sq = sum_sq + d * d;
        }
        float inv = 1.0f / std::sqrt(sum_sq / float(dim) + eps);
        for (int64_t i = 0; i < dim; ++i) {
            float v = (rs_bf16_f32(x[r * dim + i]) - mean) * inv;
            if (chain) v = rs_bf16_f32(rs_bf16_rne(v));
            if (s) v = v * (rs_bf16_f32(s[i]) + bias) + rs_bf16_f32(t[i]);
            out[r * dim + i] = rs_bf16_rne(v);
        }
    }
}

// thinfer-core/src/ops/sdpa.rs:10-47 (shapes, GQA head map, mask modes) and :131-224 (SdpaF32): scaled-dot-product
// attention with online softmax, one query row at a time, keys in ascending order:
//   s_j = dot(q, k_j) * scale + bias_j ; m' = max(m, s_j) ; alpha = exp(m - m') ; p = exp(s_j - m')
//   o = o * alpha + p * v_j ; l = l * alpha + p ; out = o / l
// with the running maximum started at -3.4e38 (finite, as the reference does for WGSL). Q [B, Sq, Hq, D],
// K / V [B, Sk, Hkv, D] (head hq reads kv head hq * Hkv / Hq), Out [B, Sq, Hq, D]; f32 arithmetic. mask_mode 0: no
// bias (mask may be null); 1: mask [B, Sq, Sk]; 2: mask [B, Hq, Sq, Sk]. bf16 != 0: tensors are bf16 bit patterns
// and the output is rounded to bf16 (the reference's act_store). Rows are independent: OpenMP over them.
void ref_sdpa(const void* q, const void* k, const void* v, const void* mask, int bf16, int64_t b, int64_t s_q, int64_t s_k,
              int64_t h_q, int64_t h_kv, int64_t d, float scale, int mask_mode, void* out) {
    auto ld = [bf16](const void* p, int64_t i) {
        return bf16 ? rs_bf16_f32(static_cast<const uint16_t*>(p)[i]) : static_cast<const float*>(p)[i];
    };
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t bb = 0; bb < b; ++bb) {
        for (int64_t sq = 0; sq < s_q; ++sq) {
            float* ql = new float[d];
            float* ol = new float[d];
            for (int64_t hq = 0; hq < h_q; ++hq) {
                const int64_t hkv = (hq * h_kv) / h_q;
                const int64_t q_off = ((bb * s_q + sq) * h_q + hq) * d;
                const int64_t kv_b0 = (bb * s_k * h_kv + hkv) * d, kv_step = h_kv * d;
                const int64_t mask_base = (mask_mode == 2 ? (bb * h_q + hq) * s_q + sq : bb * s_q + sq) * s_k;
                for (int64_t i = 0; i < d; ++i) {
                    ql[i] = ld(q, q_off + i);
                    ol[i] = 0.0f;
                }
                float m = -3.4e38f, l = 0.0f;
                for (int64_t j = 0; j < s_k; ++j) {
                    const int64_t base = kv_b0 + j * kv_step;
                    float dot = 0.0f;
                    for (int64_t i = 0; i < d; ++i) dot = dot + ql[i] * ld(k, base + i);
                    const float bias = mask_mode != 0 ? ld(mask, mask_base + j) : 0.0f;
                    const float s_j = dot * scale + bias;
                    const float m_new = std::fmax(m, s_j);
                    const float alpha = std::exp(m - m_new), p_j = std::exp(s_j - m_new);
                    for (int64_t i = 0; i < d; ++i) ol[i] = ol[i] * alpha + p_j * ld(v, base + i);
                    l = l * alpha + p_j;
                    m = m_new;
                }
                const float inv_l = 1.0f / l;
                for (int64_t i = 0; i < d; ++i) {
                    const float o = ol[i] * inv_l;
                    if (bf16) static_cast<uint16_t*>(out)[q_off + i] = rs_bf16_rne(o);
                    else static_cast<float*>(out)[q_off + i] = o;
                }
            }
            delete[] ql;
            delete[] ol;
        }
    }
}

}  // extern "C"
