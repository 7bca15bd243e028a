// TEST INFRASTRUCTURE ONLY -- CPU oracle for the FlashCK attention hot path.
//
// PARITY UNPINNED: the reference repository (Yanxing-Shi/FlashCK) holds no golden
// vector, known-answer test or fixture for its attention path (its four FMHA
// test files are empty) and its arithmetic lives in the un-vendored
// `composable_kernel` submodule (branch `develop`, commit not pinned).  This file
// therefore restates the published algorithm (scaled dot-product attention with
// fp32 accumulation) under the conventions FlashCK's own files fix:
//
//   * dtype pipeline (core/module/kernels/attention_kernels/fmha_common_jinja.h:120-155):
//     Q/K/V/P/O in fp16 or bf16; S, softmax, O accumulation and LSE in fp32;
//     LSE = max + log(sum) (natural log) of the scaled, masked scores.
//   * layouts (fmha_fwd/fmha_fwd_jinja.h:195-235): BSHD, row stride h*d, head
//     stride d; group mode packs sequences with int64 seqstart arrays
//     (fmha_fwd/fmha_fwd_call.h:14-16).
//   * GQA head map kv_head = q_head / (hq / hkv) (fmha_fwd/fmha_fwd_jinja.h:325).
//   * mask enum 0 none / 1 top-left / 2 bottom-right / 3 generic and the
//     [left,right] window with -1 = unbounded (core/profiling/attention/fmha_library.h:81-87,
//     fmha_fwd/fmha_fwd_jinja.h:299-302).
//   * paged K/V pool [num_pages, page_block_size, hkv, d] addressed through an
//     int32 block table [batch, max_pages_per_seq]
//     (fmha_fwd_split_kv/fmha_fwd_split_kv_jinja.h:296-318,512-519,550).
//   * split-KV workspaces lse_acc [b,hq,S,sq], o_acc [b,hq,S,sq,dv] fp32 and the
//     LSE-weighted combine (fmha_fwd_split_kv_jinja.h:543-547,
//     fmha_fwd_split_kv_combine/fmha_fwd_split_kv_combine_jinja.h:125-140).
//   * RoPE modes interleaved / half-rotated (fmha_library.h:195-199) with cos/sin
//     tables [positions, rotary_dim/2] in the input dtype (fmha_common_jinja.h:208-224).
//
// Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm
// may load this library, and only as the checker or the timed CPU baseline.
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

constexpr int kFloat16  = 3;  // core/utils/dtype.h:16-28 DataType::FLOAT16
constexpr int kBFloat16 = 4;  // DataType::BFLOAT16

inline float bf16_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {  // round to nearest even, NaN kept quiet
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            u = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_f16(float f) {  // round to nearest even
    uint32_t u;
    std::memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return static_cast<uint16_t>(sign | 0x7e00u);
    if (a >= 0x47800000u) return static_cast<uint16_t>(sign | 0x7c00u);  // >= 65536 -> inf (65520 rounds up too)
    if (a < 0x38800000u) {  // subnormal half or zero
        if (a < 0x33000000u) return static_cast<uint16_t>(sign);
        int e = static_cast<int>(a >> 23);
        uint32_t man = (a & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;  // 14..24
        uint32_t half = man >> shift, rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return static_cast<uint16_t>(sign | half);
    }
    uint32_t r = a + 0xfffu + ((a >> 13) & 1u);
    r = ((r >> 13) - (112u << 10));
    if (r >= 0x7c00u) r = 0x7c00u;
    return static_cast<uint16_t>(sign | r);
}
inline float to_f32(uint16_t h, int dtype) { return dtype == kBFloat16 ? bf16_to_f32(h) : f16_to_f32(h); }
inline uint16_t from_f32(float f, int dtype) { return dtype == kBFloat16 ? f32_to_bf16(f) : f32_to_f16(f); }

// Visible key range [lo, hi] (inclusive) for query row i of a (sq x sk) problem.
inline void visible_range(int64_t i, int64_t sq, int64_t sk, uint32_t mask_type, int64_t wl, int64_t wr,
                          int64_t& lo, int64_t& hi) {
    lo = 0;
    hi = sk - 1;
    if (mask_type == 0) return;
    const int64_t shift = (mask_type == 2) ? (sk - sq) : 0;  // bottom-right aligns the last query with the last key
    if (wl >= 0) lo = std::max<int64_t>(lo, i + shift - wl);
    if (wr >= 0) hi = std::min<int64_t>(hi, i + shift + wr);
}

struct KvView {
    const uint16_t* k;
    const uint16_t* v;
    const int32_t* block_table;  // nullptr => contiguous
    int64_t bt_stride;           // entries per batch row
    int64_t page;                // page_block_size
    int64_t hkv, d, dv;
    // contiguous addressing: token row index of key j
    int64_t row0;  // first token row of this sequence in the contiguous buffer
    inline int64_t token_row(int64_t b_phys, int64_t j) const {
        if (block_table) {
            const int64_t pg = block_table[b_phys * bt_stride + j / page];
            return pg * page + j % page;
        }
        return row0 + j;
    }
};

// One (sequence, q head): rows [0,sq) against keys [0,sk).
void attend_head(const uint16_t* q, int64_t q_row_stride, const KvView& kv, int64_t b_phys, int64_t kvh,
                 int64_t sq, int64_t sk, int64_t d, int64_t dv, float scale, uint32_t mask_type, int64_t wl,
                 int64_t wr, int dtype, uint16_t* o, int64_t o_row_stride, float* lse, int64_t lse_stride,
                 const float* kf, const float* vf /* fp32 copies of this kv head: [sk,d], [sk,dv] */,
                 const uint16_t* bias /* first element of this (sequence, head) block, or nullptr */,
                 int64_t bias_row_stride, float alibi_slope, float soft_cap) {
    std::vector<float> s(static_cast<size_t>(std::max<int64_t>(sk, 1)));
    std::vector<float> qf(d), acc(dv);
    for (int64_t i = 0; i < sq; ++i) {
        int64_t lo, hi;
        visible_range(i, sq, sk, mask_type, wl, wr, lo, hi);
        for (int64_t x = 0; x < d; ++x) qf[x] = to_f32(q[i * q_row_stride + x], dtype);
        float m = -std::numeric_limits<float>::infinity();
        for (int64_t j = lo; j <= hi; ++j) {
            const float* kr = kf + j * d;
            float a = 0.f;
            for (int64_t x = 0; x < d; ++x) a += qf[x] * kr[x];
            a *= scale;
            // has_logits_soft_cap (fmha_fwd/fmha_fwd_problem.h:81): the scaled score is capped, then the bias is added
            if (soft_cap > 0.f) a = soft_cap * std::tanh(a / soft_cap);
            if (bias) a += to_f32(bias[i * bias_row_stride + j], dtype);  // ELEMENTWISE_BIAS (fmha_library.h:123)
            // ALIBI (fmha_library.h:124): distance from the diagonal that ends at the last query and the last key
            if (alibi_slope != 0.f) a -= alibi_slope * std::fabs(static_cast<float>(i + sk - sq - j));
            s[j] = a;
            m = std::max(m, a);
        }
        std::fill(acc.begin(), acc.end(), 0.f);
        if (hi < lo || m == -std::numeric_limits<float>::infinity()) {  // fully masked row: O = 0, LSE = -inf
            for (int64_t x = 0; x < dv; ++x) o[i * o_row_stride + x] = from_f32(0.f, dtype);
            if (lse) lse[i * lse_stride] = -std::numeric_limits<float>::infinity();
            continue;
        }
        float l = 0.f;
        for (int64_t j = lo; j <= hi; ++j) {
            const float p = std::exp(s[j] - m);
            l += p;
            s[j] = p;
        }
        const float inv = 1.f / l;
        for (int64_t j = lo; j <= hi; ++j) {
            // P is rounded to the input dtype before the second GEMM (PDataType).
            const float p = to_f32(from_f32(s[j] * inv, dtype), dtype);
            const float* vr = vf + j * dv;
            for (int64_t x = 0; x < dv; ++x) acc[x] += p * vr[x];
        }
        for (int64_t x = 0; x < dv; ++x) o[i * o_row_stride + x] = from_f32(acc[x], dtype);
        if (lse) lse[i * lse_stride] = m + std::log(l);
    }
    (void)kv; (void)b_phys; (void)kvh;
}

}  // namespace

extern "C" {

// Dense / varlen / paged forward attention.
//   batch mode (seqstart_q == nullptr): Q [b,sq,hq,d], O [b,sq,hq,dv], LSE [b,hq,sq].
//   group mode: Q [total_q,hq,d], O [total_q,hq,dv], LSE [hq,total_q]; seqstart_q/k int64 [b+1].
//   K/V contiguous: batch mode [b,sk,hkv,d]; group mode [total_k,hkv,d] (seqstart_k), or, when
//   seqstart_k == nullptr in group mode, batch-strided [b,sk,hkv,d] with per-batch seqlen_k.
//   K/V paged (block_table != nullptr): pool [pages,page,hkv,d]; per-batch lengths in seqlen_k (int32).
//   cache_batch_idx (int64 [b], optional) remaps the batch row used for K/V and the block table.
// bias_enum / bias_rank_info as in fmha_library.h:121-164 and the strides of fmha_fwd/fmha_fwd_jinja.h:199-233,
// 270-293: elementwise bias in the element dtype, rank 0 = [1,1,sq,sk], 1 = [1,hq,sq,sk], 2 = [b,hq,sq,sk] (group
// mode: sq, sk are the packed totals, a sequence's block starts at its first packed row and key); ALiBi slopes fp32,
// rank 0 = [1,hq], 1 = [b,hq].  The ALiBi term itself is computed inside ck_tile, which is not part of the reference
// tree: the form used here is the published one with the diagonal aligned bottom-right.
int oracle_fmha_fwd_bias(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* o, float* lse,
                         const int64_t* seqstart_q, const int64_t* seqstart_k, const int32_t* seqlen_k_ptr,
                         const int32_t* block_table, const int64_t* cache_batch_idx, int64_t batch, int64_t seqlen_q,
                         int64_t seqlen_k, int64_t hq, int64_t hkv, int64_t d, int64_t dv, int64_t bt_stride,
                         int64_t page_block_size, float scale, int64_t window_left, int64_t window_right,
                         uint32_t mask_type, int dtype, int nthreads, const void* bias, int bias_enum,
                         int bias_rank_info, float logits_soft_cap) {
    if (hq % hkv != 0 || (dtype != kFloat16 && dtype != kBFloat16)) return 1;
    if (scale == 0.f) scale = 1.f / std::sqrt(static_cast<float>(d));  // fmha_fwd_jinja.h:57-59
    const int64_t ratio = hq / hkv;
    const int64_t total_q = seqstart_q ? seqstart_q[batch] : batch * seqlen_q;
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t kh = 0; kh < hkv; ++kh) {
            const int64_t q0 = seqstart_q ? seqstart_q[b] : b * seqlen_q;
            const int64_t sq = seqstart_q ? seqstart_q[b + 1] - seqstart_q[b] : seqlen_q;
            int64_t sk;
            if (seqlen_k_ptr) sk = seqlen_k_ptr[b];
            else if (seqstart_k) sk = seqstart_k[b + 1] - seqstart_k[b];
            else sk = seqlen_k;
            const int64_t b_phys = cache_batch_idx ? cache_batch_idx[b] : b;
            KvView kv{k, v, block_table, bt_stride, page_block_size, hkv, d, dv,
                      seqstart_k ? seqstart_k[b] : b_phys * seqlen_k};
            std::vector<float> kf(static_cast<size_t>(std::max<int64_t>(sk, 1) * d));
            std::vector<float> vf(static_cast<size_t>(std::max<int64_t>(sk, 1) * dv));
            for (int64_t j = 0; j < sk; ++j) {
                const int64_t r = kv.token_row(b_phys, j);
                const uint16_t* kr = k + (r * hkv + kh) * d;
                const uint16_t* vr = v + (r * hkv + kh) * dv;
                for (int64_t x = 0; x < d; ++x) kf[j * d + x] = to_f32(kr[x], dtype);
                for (int64_t x = 0; x < dv; ++x) vf[j * dv + x] = to_f32(vr[x], dtype);
            }
            for (int64_t g = 0; g < ratio; ++g) {
                const int64_t h = kh * ratio + g;
                float* lse_h = nullptr;
                int64_t lse_stride = 1;
                if (lse) lse_h = seqstart_q ? lse + h * total_q + q0 : lse + (b * hq + h) * seqlen_q;
                const uint16_t* bias_blk = nullptr;
                float slope = 0.f;
                const int64_t plane_sq = seqstart_q ? total_q : seqlen_q, plane_sk = seqlen_k;
                if (bias && bias_enum == 1) {
                    const int64_t plane = plane_sq * plane_sk;
                    int64_t off = bias_rank_info >= 1 ? h * plane : 0;
                    if (bias_rank_info == 2 && !seqstart_q) off += b * hq * plane;
                    if (seqstart_q) off += q0 * plane_sk + (seqstart_k ? seqstart_k[b] : 0);
                    bias_blk = static_cast<const uint16_t*>(bias) + off;
                } else if (bias && bias_enum == 2) {
                    slope = static_cast<const float*>(bias)[(bias_rank_info >= 1 ? b * hq : 0) + h];
                }
                attend_head(q + (q0 * hq + h) * d, hq * d, kv, b_phys, kh, sq, sk, d, dv, scale, mask_type,
                            window_left, window_right, dtype, o + (q0 * hq + h) * dv, hq * dv, lse_h, lse_stride,
                            kf.data(), vf.data(), bias_blk, plane_sk, slope, logits_soft_cap);
            }
        }
    }
    return 0;
}

int oracle_fmha_fwd(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* o, float* lse,
                    const int64_t* seqstart_q, const int64_t* seqstart_k, const int32_t* seqlen_k_ptr,
                    const int32_t* block_table, const int64_t* cache_batch_idx, int64_t batch, int64_t seqlen_q,
                    int64_t seqlen_k, int64_t hq, int64_t hkv, int64_t d, int64_t dv, int64_t bt_stride,
                    int64_t page_block_size, float scale, int64_t window_left, int64_t window_right,
                    uint32_t mask_type, int dtype, int nthreads) {
    return oracle_fmha_fwd_bias(q, k, v, o, lse, seqstart_q, seqstart_k, seqlen_k_ptr, block_table, cache_batch_idx, batch,
                                seqlen_q, seqlen_k, hq, hkv, d, dv, bt_stride, page_block_size, scale, window_left,
                                window_right, mask_type, dtype, nthreads, nullptr, 0, 0, 0.f);
}

// LSE-weighted combine of split-KV partials (fmha_fwd_split_kv_combine_jinja.h:125-140):
//   lse_acc [bs,hq,S,rows], o_acc [bs,hq,S,rows,dv] fp32 -> O [bs,rows,hq,dv] (dtype), LSE [bs,hq,rows].
//   (group mode: bs = 1 and rows = total_q.)  A split with LSE = -inf has weight 0.
int oracle_splitkv_combine(const float* lse_acc, const float* o_acc, uint16_t* o, float* lse, int64_t bs,
                           int64_t rows, int64_t hq, int64_t dv, int64_t num_splits, int dtype) {
    const float ninf = -std::numeric_limits<float>::infinity();
#pragma omp parallel for collapse(2)
    for (int64_t b = 0; b < bs; ++b)
        for (int64_t h = 0; h < hq; ++h)
            for (int64_t r = 0; r < rows; ++r) {
                float m = ninf;
                for (int64_t s = 0; s < num_splits; ++s)
                    m = std::max(m, lse_acc[((b * hq + h) * num_splits + s) * rows + r]);
                uint16_t* orow = o + ((b * rows + r) * hq + h) * dv;
                if (m == ninf) {
                    for (int64_t x = 0; x < dv; ++x) orow[x] = from_f32(0.f, dtype);
                    if (lse) lse[(b * hq + h) * rows + r] = ninf;
                    continue;
                }
                std::vector<float> acc(dv, 0.f);
                float sum = 0.f;
                for (int64_t s = 0; s < num_splits; ++s) {
                    const float ls = lse_acc[((b * hq + h) * num_splits + s) * rows + r];
                    if (ls == ninf) continue;
                    const float w = std::exp(ls - m);
                    sum += w;
                    const float* oa = o_acc + (((b * hq + h) * num_splits + s) * rows + r) * dv;
                    for (int64_t x = 0; x < dv; ++x) acc[x] += w * oa[x];
                }
                for (int64_t x = 0; x < dv; ++x) orow[x] = from_f32(acc[x] / sum, dtype);
                if (lse) lse[(b * hq + h) * rows + r] = m + std::log(sum);
            }
    return 0;
}

int oracle_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
