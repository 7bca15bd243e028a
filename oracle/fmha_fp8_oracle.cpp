// TEST INFRASTRUCTURE ONLY -- CPU oracle for the 8-bit (static-quantisation) forward attention.
//
// PARITY UNPINNED, like fmha_oracle.cpp: the reference holds no golden vector for this path and the arithmetic lives
// in the absent ck_tile submodule.  What the reference's own files fix, and this file follows:
//   * the type pipeline FmhaFwdTypeConfig<fp8_t / bf8_t> (core/module/kernels/attention_kernels/
//     fmha_common_jinja.h:157-187): Q, K, V, P and O are 8-bit floats; S, the softmax, the O accumulator and the LSE
//     are fp32;
//   * the three static scales of the kernel arguments, scale_s, scale_p, scale_o (fmha_fwd/fmha_fwd_jinja.h:93,
//     326-328; fmha_fwd_split_kv/fmha_fwd_split_kv_jinja.h:116-118): scale_s multiplies Q K^T (softmax scale times the
//     de-quantisation of Q and K), scale_p stretches the probabilities over the 8-bit range before they are rounded for
//     the second GEMM, scale_o takes the accumulator back to the range of O;
//   * DataType codes 1 = FLOAT8, 2 = BFLOAT8 (core/utils/dtype.h:16-28).
// The 8-bit formats are the OCP ones a B200 computes in: FLOAT8 = E4M3 (bias 7, max 448, no infinity), BFLOAT8 = E5M2
// (bias 15, max 57344).  Conversions round to nearest even and saturate to the largest finite value.
//
// Restated algorithm, per query row i (fp32 arithmetic unless stated):
//     s_j = scale_s * sum_x q_ix k_jx  (masked keys dropped);   m = max_j s_j;   p_j = exp(s_j - m);   l = sum_j p_j
//     P8_j = round_to_8bit(scale_p * p_j);   acc = sum_j P8_j * v_j;   O_i = round_to_out(scale_o * acc / l)
//     LSE_i = m + log(l)
// A kernel that works tile by tile rounds p_j relative to a running maximum instead of the final one; both are roundings
// of the same quantity to 3 (E4M3) or 2 (E5M2) mantissa bits, so results agree to the precision of P8, not bit for bit.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr int kFloat8 = 1, kBFloat8 = 2, kFloat16 = 3, kBFloat16 = 4;

// Generic small-float decode / encode: `eb` exponent bits, `mb` mantissa bits, bias 2^(eb-1) - 1.
// E4M3 (finite-only): the all-ones exponent holds ordinary numbers except mantissa 111 (NaN).  E5M2: IEEE-like.
inline float f8_to_f32(uint8_t h, int dtype) {
    const int eb = dtype == kFloat8 ? 4 : 5, mb = 7 - eb, bias = (1 << (eb - 1)) - 1;
    const int sign = h >> 7, e = (h >> mb) & ((1 << eb) - 1), m = h & ((1 << mb) - 1);
    float v;
    if (dtype == kFloat8 && e == 15 && m == 7) v = std::numeric_limits<float>::quiet_NaN();
    else if (dtype == kBFloat8 && e == 31) v = m ? std::numeric_limits<float>::quiet_NaN() : std::numeric_limits<float>::infinity();
    else if (e == 0) v = std::ldexp(static_cast<float>(m), 1 - bias - mb);
    else v = std::ldexp(static_cast<float>((1 << mb) | m), e - bias - mb);
    return sign ? -v : v;
}
inline uint8_t f32_to_f8(float f, int dtype) {  // round to nearest even, saturate to the largest finite value
    const int eb = dtype == kFloat8 ? 4 : 5, mb = 7 - eb, bias = (1 << (eb - 1)) - 1;
    const float fmax = dtype == kFloat8 ? 448.f : 57344.f;
    const uint8_t sign = std::signbit(f) ? 0x80 : 0;
    if (std::isnan(f)) return sign | 0x7f;
    float a = std::fabs(f);
    if (a >= fmax) return sign | (dtype == kFloat8 ? 0x7e : 0x7b);
    if (a == 0.f) return sign;
    int ex;
    std::frexp(a, &ex);                 // a = frac * 2^ex, frac in [0.5, 1)
    int e = ex - 1;                     // a = 1.xxx * 2^e
    const int emin = 1 - bias;          // exponent of the smallest normal
    const int q = std::max(e, emin) - mb;  // weight of the last kept bit
    const float scaled = std::ldexp(a, -q);
    float r = std::nearbyint(scaled);   // default rounding mode: to nearest even
    float back = std::ldexp(r, q);
    if (back >= fmax) return sign | (dtype == kFloat8 ? 0x7e : 0x7b);
    if (back == 0.f) return sign;
    std::frexp(back, &ex);
    e = ex - 1;
    if (e < emin) {                     // subnormal
        const int m = static_cast<int>(std::ldexp(back, -(emin - mb)));
        return sign | static_cast<uint8_t>(m);
    }
    const int m = static_cast<int>(std::ldexp(back, -(e - mb))) - (1 << mb);
    return sign | static_cast<uint8_t>(((e + bias) << mb) | m);
}

inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
inline uint16_t f32_to_f16(float f) {  // through the 8 + 10 bit split: exact for the magnitudes an O row takes
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return static_cast<uint16_t>(sign | 0x7e00u);
    if (a >= 0x47800000u) return static_cast<uint16_t>(sign | 0x7c00u);
    if (a < 0x38800000u) {
        if (a < 0x33000000u) return static_cast<uint16_t>(sign);
        const int e = static_cast<int>(a >> 23);
        const uint32_t man = (a & 0x7fffffu) | 0x800000u;
        const int shift = 126 - e;
        uint32_t half = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return static_cast<uint16_t>(sign | half);
    }
    uint32_t r = a + 0xfffu + ((a >> 13) & 1u);
    r = (r >> 13) - (112u << 10);
    if (r >= 0x7c00u) r = 0x7c00u;
    return static_cast<uint16_t>(sign | r);
}

inline void visible_range(int64_t i, int64_t sq, int64_t sk, uint32_t mask_type, int64_t wl, int64_t wr, int64_t& lo, int64_t& hi) {
    lo = 0;
    hi = sk - 1;
    if (mask_type == 0) return;
    const int64_t shift = (mask_type == 2) ? (sk - sq) : 0;
    if (wl >= 0) lo = std::max<int64_t>(lo, i + shift - wl);
    if (wr >= 0) hi = std::min<int64_t>(hi, i + shift + wr);
}

}  // namespace

extern "C" {

// Element conversions, exported so that the tests can pin them against an independent implementation.
float oracle_f8_to_f32(uint8_t h, int dtype) { return f8_to_f32(h, dtype); }
uint8_t oracle_f32_to_f8(float f, int dtype) { return f32_to_f8(f, dtype); }

// Batch mode (seqstart_q == nullptr): Q [b,sq,hq,d], K [b,sk,hkv,d], V [b,sk,hkv,dv]; group mode: packed tokens with
// int64 seqstart arrays.  dtype 1 (E4M3) or 2 (E5M2) for Q/K/V/P; out_dtype 1, 2 (one byte per element), 3 or 4 (two).
int oracle_fmha_fwd_fp8(const uint8_t* q, const uint8_t* k, const uint8_t* v, void* o, float* lse, const int64_t* seqstart_q,
                        const int64_t* seqstart_k, int64_t batch, int64_t seqlen_q, int64_t seqlen_k, int64_t hq, int64_t hkv,
                        int64_t d, int64_t dv, float scale_s, float scale_p, float scale_o, int64_t window_left,
                        int64_t window_right, uint32_t mask_type, int dtype, int out_dtype, int nthreads) {
    if (hq % hkv != 0 || (dtype != kFloat8 && dtype != kBFloat8) || out_dtype < 1 || out_dtype > 4) return 1;
    const int64_t ratio = hq / hkv;
    const int64_t total_q = seqstart_q ? seqstart_q[batch] : batch * seqlen_q;
    const float ninf = -std::numeric_limits<float>::infinity();
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t h = 0; h < hq; ++h) {
            const int64_t kh = h / ratio;
            const int64_t q0 = seqstart_q ? seqstart_q[b] : b * seqlen_q;
            const int64_t sq = seqstart_q ? seqstart_q[b + 1] - seqstart_q[b] : seqlen_q;
            const int64_t k0 = seqstart_k ? seqstart_k[b] : b * seqlen_k;
            const int64_t sk = seqstart_k ? seqstart_k[b + 1] - seqstart_k[b] : seqlen_k;
            std::vector<float> kf(static_cast<size_t>(std::max<int64_t>(sk, 1) * d)), vf(static_cast<size_t>(std::max<int64_t>(sk, 1) * dv));
            for (int64_t j = 0; j < sk; ++j) {
                for (int64_t x = 0; x < d; ++x) kf[j * d + x] = f8_to_f32(k[((k0 + j) * hkv + kh) * d + x], dtype);
                for (int64_t x = 0; x < dv; ++x) vf[j * dv + x] = f8_to_f32(v[((k0 + j) * hkv + kh) * dv + x], dtype);
            }
            std::vector<float> s(static_cast<size_t>(std::max<int64_t>(sk, 1))), qf(d), acc(dv);
            for (int64_t i = 0; i < sq; ++i) {
                int64_t lo, hi;
                visible_range(i, sq, sk, mask_type, window_left, window_right, lo, hi);
                for (int64_t x = 0; x < d; ++x) qf[x] = f8_to_f32(q[((q0 + i) * hq + h) * d + x], dtype);
                float m = ninf;
                for (int64_t j = lo; j <= hi; ++j) {
                    float a = 0.f;
                    for (int64_t x = 0; x < d; ++x) a += qf[x] * kf[j * d + x];
                    s[j] = a * scale_s;
                    m = std::max(m, s[j]);
                }
                std::fill(acc.begin(), acc.end(), 0.f);
                float l = 0.f;
                if (hi >= lo && m != ninf) {
                    for (int64_t j = lo; j <= hi; ++j) {
                        const float p = std::exp(s[j] - m);
                        l += p;
                        const float p8 = f8_to_f32(f32_to_f8(scale_p * p, dtype), dtype);  // PDataType is the 8-bit type
                        for (int64_t x = 0; x < dv; ++x) acc[x] += p8 * vf[j * dv + x];
                    }
                }
                const int64_t orow = ((q0 + i) * hq + h) * dv;
                for (int64_t x = 0; x < dv; ++x) {
                    const float val = l > 0.f ? scale_o * acc[x] / l : 0.f;
                    if (out_dtype <= 2) static_cast<uint8_t*>(o)[orow + x] = f32_to_f8(val, out_dtype);
                    else static_cast<uint16_t*>(o)[orow + x] = out_dtype == kBFloat16 ? f32_to_bf16(val) : f32_to_f16(val);
                }
                if (lse) {
                    float* lp = seqstart_q ? lse + h * total_q + q0 + i : lse + (b * hq + h) * seqlen_q + i;
                    *lp = l > 0.f ? m + std::log(l) : ninf;
                }
            }
        }
    }
    return 0;
}

}  // extern "C"
