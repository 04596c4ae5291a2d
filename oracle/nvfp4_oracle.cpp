// TEST INFRASTRUCTURE — CPU oracle for the NVFP4 linear path. Not a product path.
//
// Only the test-suite, the smoke check and the bench's CPU-baseline leg may load this
// library; the shipped library never links or calls it.
//
// PARITY STATUS: "parity unpinned" for the NVFP4 arithmetic itself. The reference
// (cretz/thinfer) has no FP4/E4M3 quantiser, kernel, test or fixture, so nothing in it
// fixes an E2M1 code, an E4M3 block scale or an FP4 GEMM result. What IS pinned by the
// reference and re-used here: bf16 round-to-nearest-even (thinfer-core/src/ops/mod.rs:556-561,
// thinfer-core/src/ops/weight_prep.rs:196-207), the f32 K-ascending accumulate order of its
// CPU linear (thinfer-conformance/tests/q4_0_matmul.rs:23-43), bias add then round
// (thinfer-core/src/ops/bcast_add.rs), tanh-GELU constants (thinfer-core/src/ops/gelu.rs:21-31),
// "store the block parameters at storage precision first, then compute codes against the
// stored value" (thinfer-core/src/ops/act_quant.rs:121-151) and "all-zero block -> zero
// scale, zero codes" (thinfer-core/src/quant.rs:186-188,747). Those shared pieces are checked
// against the reference's committed fixtures and unit-test properties in tests/.
//
// The NVFP4 format restated here is the published one: E2M1 elements
// (+-{0,0.5,1,1.5,2,3,4,6}), two per byte with the even K index in the low nibble, one
// unsigned E4M3 scale per 16 consecutive K elements, one FP32 scale per tensor.
//
// Build: see oracle/Makefile (g++ -O3 -march=x86-64-v3 -fopenmp -ffp-contract=off).
// -ffp-contract=off matters: every f32 operation below is a separately rounded IEEE
// operation, which is what the CUDA kernels reproduce with __fmul_rn/__fdiv_rn.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline uint32_t f32_bits(float x) { uint32_t b; std::memcpy(&b, &x, 4); return b; }
inline float bits_f32(uint32_t b) { float x; std::memcpy(&x, &b, 4); return x; }

// bf16 RNE with NaN quieting. Follows thinfer-core/src/ops/weight_prep.rs:201-207
// (bit-exact with half::bf16::from_f32 per that file's comment).
inline uint16_t bf16_rne(float x) {
    uint32_t b = f32_bits(x);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((b >> 16) | 0x40u);
    if ((b & 0x8000u) != 0u && (b & 0x17FFFu) != 0u) return uint16_t(((b >> 16) + 1u) & 0xFFFFu);
    return uint16_t(b >> 16);
}
inline float bf16_f32(uint16_t h) { return bits_f32(uint32_t(h) << 16); }

// Unsigned E4M3 (fn variant: bias 7, max finite 448 = 0x7E, 0x7F = NaN), RNE,
// saturating to 448. Input is expected >= 0.
inline uint8_t e4m3_encode(float x) {
    if (x != x) return 0x7F;
    if (!(x > 0.0f)) return 0;
    if (x > 448.0f) return 0x7E;
    uint32_t b = f32_bits(x);
    int e = int((b >> 23) & 0xFF) - 127;
    if (e < -6) {
        // subnormal range of the target: multiples of 2^-9; x*512 is exact (power of two)
        float q = std::nearbyintf(x * 512.0f);  // default rounding mode = ties to even
        return uint8_t(int(q));                 // 8 encodes the smallest normal, 2^-6
    }
    uint32_t mant = b & 0x7FFFFFu;
    uint32_t m = mant >> 20, rem = mant & 0xFFFFFu;
    if (rem > 0x80000u || (rem == 0x80000u && (m & 1u))) m += 1;
    if (m == 8) { m = 0; e += 1; }
    uint32_t code = (uint32_t(e + 7) << 3) | m;
    return uint8_t(code > 0x7Eu ? 0x7Eu : code);
}
inline float e4m3_decode(uint8_t c) {
    int e = (c >> 3) & 0xF, m = c & 7;
    if (e == 0xF && m == 7) return NAN;
    float v = (e == 0) ? std::ldexp(float(m), -9) : std::ldexp(float(8 + m), e - 10);
    return (c & 0x80) ? -v : v;
}

// E2M1 RNE, saturating at +-6, ties to the even code; the sign bit (bit 3) is kept even
// when the magnitude rounds to zero. NaN -> +6 (code 7).
inline uint8_t e2m1_encode(float y) {
    if (y != y) return 7;
    uint8_t s = (f32_bits(y) >> 31) ? 8 : 0;
    float a = std::fabs(y);
    uint8_t c;
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return s | c;
}
const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
inline float e2m1_decode(uint8_t c) { float v = kE2M1[c & 7]; return (c & 8) ? -v : v; }

// One 16-element block. `x` already f32. Writes 8 code bytes and returns the scale byte.
inline uint8_t quant_block16(const float* x, float g, uint8_t* codes8) {
    float bmax = 0.0f;
    for (int i = 0; i < 16; ++i) bmax = std::fmax(bmax, std::fabs(x[i]));
    float t = 6.0f * g;
    float inv_t = 1.0f / t;
    float s_raw = bmax * inv_t;
    uint8_t sc = e4m3_encode(s_raw);
    if (sc == 0 || sc == 0x7F) {
        // degenerate block: zero scale -> zero codes (thinfer-core/src/quant.rs:186-188 idea)
        for (int i = 0; i < 8; ++i) codes8[i] = 0;
        return sc == 0x7F ? 0 : sc;
    }
    float d = e4m3_decode(sc) * g;   // stored-precision scale, as act_quant.rs:137-143 does
    float inv_d = 1.0f / d;
    for (int i = 0; i < 8; ++i) {
        uint8_t lo = e2m1_encode(x[2 * i] * inv_d);
        uint8_t hi = e2m1_encode(x[2 * i + 1] * inv_d);
        codes8[i] = uint8_t(lo | (hi << 4));
    }
    return sc;
}

inline float gelu_tanh(float x) {
    // thinfer-core/src/ops/gelu.rs:21-31
    const float c = 0.7978845608028654f;
    float inner = c * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + std::tanh(inner));
}

}  // namespace

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// A launcher may have pinned OMP_NUM_THREADS to 1 for its workers; the timed CPU leg sets the count itself.
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

uint16_t orc_bf16_rne(float x) { return bf16_rne(x); }
float orc_bf16_to_f32(uint16_t h) { return bf16_f32(h); }
uint8_t orc_e4m3_encode(float x) { return e4m3_encode(x); }
float orc_e4m3_decode(uint8_t c) { return e4m3_decode(c); }
uint8_t orc_e2m1_encode(float x) { return e2m1_encode(x); }
float orc_e2m1_decode(uint8_t c) { return e2m1_decode(c); }

void orc_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[i] = bf16_rne(src[i]);
}

// SplitMix64 -> Box-Muller standard normals, restating
// thinfer-models/src/wan/pipeline.rs:2203-2224 (gaussian_noise).
void orc_gaussian(float* out, int64_t n, uint64_t seed) {
    uint64_t state = seed + 0x9E3779B97F4A7C15ull;
    auto next = [&]() {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    };
    int64_t i = 0;
    while (i < n) {
        double u1 = (double(next() >> 11) + 1.0) * (1.0 / (double(1ull << 53) + 1.0));
        double u2 = double(next() >> 11) * (1.0 / double(1ull << 53));
        double r = std::sqrt(-2.0 * std::log(u1));
        double th = 2.0 * M_PI * u2;
        out[i++] = float(r * std::cos(th));
        if (i < n) out[i++] = float(r * std::sin(th));
    }
}

// out[i] = bf16(gaussian * sigma); convenience for the synthetic inputs.
void orc_gaussian_scaled(float* out, int64_t n, uint64_t seed, float sigma) {
    orc_gaussian(out, n, seed);
    for (int64_t i = 0; i < n; ++i) out[i] = out[i] * sigma;
}

float orc_amax_f32(const float* x, int64_t n) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) schedule(static)
    for (int64_t i = 0; i < n; ++i) m = std::fmax(m, std::fabs(x[i]));
    return m;
}
float orc_amax_bf16(const uint16_t* x, int64_t n) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) schedule(static)
    for (int64_t i = 0; i < n; ++i) m = std::fmax(m, std::fabs(bf16_f32(x[i])));
    return m;
}

// Per-tensor scale from an absolute maximum: amax / (6 * 448); 1.0 for an all-zero tensor.
float orc_global_scale(float amax) { return amax > 0.0f ? amax / 2688.0f : 1.0f; }

// Weight quantiser. w: f32 [rows, k] row-major, k % 16 == 0. codes: [rows, k/2],
// scales: [rows, k/16] (canonical row-major layouts). Returns the per-tensor scale.
float orc_quantize_weight(const float* w, int64_t rows, int64_t k, uint8_t* codes, uint8_t* scales) {
    float g = orc_global_scale(orc_amax_f32(w, rows * k));
    int64_t nb = k / 16;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b)
            scales[r * nb + b] = quant_block16(w + r * k + b * 16, g, codes + r * (k / 2) + b * 8);
    return g;
}

// Same, with the source given as bf16 bits.
float orc_quantize_weight_bf16(const uint16_t* w, int64_t rows, int64_t k, uint8_t* codes, uint8_t* scales) {
    float g = orc_global_scale(orc_amax_bf16(w, rows * k));
    int64_t nb = k / 16;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            float x[16];
            for (int i = 0; i < 16; ++i) x[i] = bf16_f32(w[r * k + b * 16 + i]);
            scales[r * nb + b] = quant_block16(x, g, codes + r * (k / 2) + b * 8);
        }
    return g;
}

// Activation quantiser: bf16 [m, k] with a GIVEN per-tensor scale g (g > 0).
void orc_quantize_act(const uint16_t* a, int64_t m, int64_t k, float g, uint8_t* codes, uint8_t* scales) {
    int64_t nb = k / 16;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < m; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            float x[16];
            for (int i = 0; i < 16; ++i) x[i] = bf16_f32(a[r * k + b * 16 + i]);
            scales[r * nb + b] = quant_block16(x, g, codes + r * (k / 2) + b * 8);
        }
}

// Dequantise canonical NVFP4 to f32 [rows, k]: code * (e4m3(scale) * g).
void orc_dequant(const uint8_t* codes, const uint8_t* scales, float g, int64_t rows, int64_t k, float* out) {
    int64_t nb = k / 16;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            float d = e4m3_decode(scales[r * nb + b]) * g;
            for (int i = 0; i < 8; ++i) {
                uint8_t by = codes[r * (k / 2) + b * 8 + i];
                out[r * k + b * 16 + 2 * i] = e2m1_decode(by & 0xF) * d;
                out[r * k + b * 16 + 2 * i + 1] = e2m1_decode(by >> 4) * d;
            }
        }
}

// Canonical [rows, k/16] scales -> the 128x4 tiled device layout consumed by the
// block-scaled MMA: 512-byte atoms indexed [row/128][kblk/4]; inside an atom the byte
// for (row r, block b) sits at (r%32)*16 + ((r%128)/32)*4 + (b%4). Rows and blocks are
// padded with zero bytes up to a multiple of 128; the atoms along K number ceil(K/64)
// rounded up to a multiple of 4 (a 256-element K tile reads four whole atoms). Returns bytes written.
int64_t orc_scales_to_device_layout(const uint8_t* scales, int64_t rows, int64_t nb, uint8_t* out) {
    int64_t rt = (rows + 127) / 128, kt = (((nb + 3) / 4) + 3) / 4 * 4;
    std::memset(out, 0, size_t(rt * kt * 512));
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            int64_t atom = (r / 128) * kt + (b / 4);
            int64_t off = atom * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4);
            out[off] = scales[r * nb + b];
        }
    return rt * kt * 512;
}

// f32 GEMM out[m,n] = sum_k a[m,k]*w[n,k], K ascending, one rounding per multiply and per
// add (the reference CPU linear, thinfer-conformance/tests/q4_0_matmul.rs:33-41). Vectorised
// across n through a transposed copy of w, which leaves each (m,n) sum order unchanged.
void orc_gemm_f32(const float* a, const float* w, int64_t m, int64_t n, int64_t k, float* out) {
    std::vector<float> wt(size_t(k) * size_t(n));
#pragma omp parallel for schedule(static)
    for (int64_t kk = 0; kk < k; ++kk)
        for (int64_t j = 0; j < n; ++j) wt[size_t(kk) * n + j] = w[size_t(j) * k + kk];
    const int64_t NB = 64;  // 8 AVX2 accumulators stay in registers
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j0 = 0; j0 < n; j0 += NB) {
            int64_t jn = std::min(NB, n - j0);
            float acc[NB];
            for (int64_t j = 0; j < jn; ++j) acc[j] = 0.0f;
            const float* ar = a + size_t(i) * k;
            for (int64_t kk = 0; kk < k; ++kk) {
                float av = ar[kk];
                const float* wr = wt.data() + size_t(kk) * n + j0;
                for (int64_t j = 0; j < jn; ++j) acc[j] = acc[j] + av * wr[j];
            }
            for (int64_t j = 0; j < jn; ++j) out[size_t(i) * n + j0 + j] = acc[j];
        }
}

// f64-accumulate variant, for error budgeting only.
void orc_gemm_f64(const float* a, const float* w, int64_t m, int64_t n, int64_t k, double* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (int64_t kk = 0; kk < k; ++kk) acc += double(a[i * k + kk]) * double(w[j * k + kk]);
            out[i * n + j] = acc;
        }
}

// Epilogue on an f32 accumulator matrix acc[m, n] (already including both per-tensor
// scales when scale == 1, otherwise multiplied by `scale` first):
//   v = acc*scale (+ bias[n]) ; act: 0 none, 1 tanh-GELU ; then, when gate != null,
//   v = residual[m,n] + gate[n]*v ; out = bf16_rne(v).
// chain != 0 inserts the reference's intermediate bf16 roundings (after the matmul, after
// the bias add, after the activation), as its separate dispatches do
// (thinfer-models/src/qwen_image/dit.rs:324-340,745-754).
void orc_epilogue(const float* acc, int64_t m, int64_t n, float scale, const uint16_t* bias,
                  int act, const uint16_t* gate, const uint16_t* residual, int chain, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            float v = acc[i * n + j] * scale;
            if (chain) v = bf16_f32(bf16_rne(v));
            if (bias) { v = v + bf16_f32(bias[j]); if (chain) v = bf16_f32(bf16_rne(v)); }
            if (act == 1) { v = gelu_tanh(v); if (chain) v = bf16_f32(bf16_rne(v)); }
            if (gate) v = bf16_f32(residual[i * n + j]) + bf16_f32(gate[j]) * v;
            out[i * n + j] = bf16_rne(v);
        }
}

// The whole linear as the device computes it: quantise A (bf16 [m,k]) with scale g_a,
// dequantise A and W to f32 WITHOUT the per-tensor scales, f32 GEMM, epilogue with
// scale = g_a*g_w. quantize_a == 0 skips the activation quantiser (bf16 activations
// against dequantised weights: the reference's own dequant-once linear).
void orc_linear(const uint16_t* a, int64_t m, int64_t k, float g_a, int quantize_a,
                const uint8_t* w_codes, const uint8_t* w_scales, float g_w, int64_t n,
                const uint16_t* bias, int act, const uint16_t* gate, const uint16_t* residual,
                int chain, uint16_t* out, float* acc_out /* optional [m,n] */) {
    std::vector<float> af(size_t(m) * k), wf(size_t(n) * k), acc(size_t(m) * n);
    float scale;
    if (quantize_a) {
        std::vector<uint8_t> ac(size_t(m) * k / 2), as(size_t(m) * k / 16);
        orc_quantize_act(a, m, k, g_a, ac.data(), as.data());
        orc_dequant(ac.data(), as.data(), 1.0f, m, k, af.data());
        scale = g_a * g_w;
    } else {
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m * k; ++i) af[i] = bf16_f32(a[i]);
        scale = g_w;
    }
    orc_dequant(w_codes, w_scales, 1.0f, n, k, wf.data());
    orc_gemm_f32(af.data(), wf.data(), m, n, k, acc.data());
    if (acc_out) std::memcpy(acc_out, acc.data(), sizeof(float) * size_t(m) * n);
    orc_epilogue(acc.data(), m, n, scale, bias, act, gate, residual, chain, out);
}

// The same linear on an activation operand that is ALREADY NVFP4 (canonical codes [m,k/2] and scales
// [m,k/16] with per-tensor scale g_a): what tnf_gemm_nvfp4 computes when the producing GEMM's epilogue
// emitted its output quantised.
void orc_linear_q(const uint8_t* a_codes, const uint8_t* a_scales, int64_t m, int64_t k, float g_a,
                  const uint8_t* w_codes, const uint8_t* w_scales, float g_w, int64_t n, const uint16_t* bias,
                  int act, const uint16_t* gate, const uint16_t* residual, int chain, uint16_t* out) {
    std::vector<float> af(size_t(m) * k), wf(size_t(n) * k), acc(size_t(m) * n);
    orc_dequant(a_codes, a_scales, 1.0f, m, k, af.data());
    orc_dequant(w_codes, w_scales, 1.0f, n, k, wf.data());
    orc_gemm_f32(af.data(), wf.data(), m, n, k, acc.data());
    orc_epilogue(acc.data(), m, n, g_a * g_w, bias, act, gate, residual, chain, out);
}

}  // extern "C"
